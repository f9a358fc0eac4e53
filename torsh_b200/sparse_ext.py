"""Sparse linear algebra, IO, analysis, layers and optimizers on top of :mod:`torsh_b200.sparse`
(``crates/torsh-sparse/src/{ops,linalg,ops_linalg,matrix_market,scipy_sparse,matlab_compat,pattern_analysis,hybrid,symmetric,
unified_interface,memory_management,optimizers}.rs`` and ``nn/``): sparse-sparse arithmetic, triangular solves, incomplete LU
and Cholesky, preconditioned CG / BiCGStab / GMRES, reverse Cuthill-McKee reordering, Matrix Market / SciPy / MATLAB
exchange, pattern statistics with format advice, hybrid and symmetric containers, sparse activations / normalisation /
pooling / attention / embedding layers, and optimizers that touch only the rows that received gradient."""
from __future__ import annotations

import math
from collections import deque
from pathlib import Path

import numpy as np
import torch
from torch import nn

from .sparse import CooTensor, CsrTensor


# ================================================================================================ arithmetic
def sparse_add(a: CooTensor, b: CooTensor, alpha: float = 1.0) -> CooTensor:
    return CooTensor(torch.cat([a.rows, b.rows]), torch.cat([a.cols, b.cols]), torch.cat([a.values, alpha * b.values]), a.shape).coalesce()


def sparse_mul(a: CooTensor, b: CooTensor) -> CooTensor:
    """Element-wise product: entries present in both."""
    a, b = a.coalesce(), b.coalesce()
    ka, kb = a.rows * a.shape[1] + a.cols, b.rows * b.shape[1] + b.cols
    pos = torch.searchsorted(kb, ka).clamp(max=max(len(kb) - 1, 0))
    hit = kb[pos] == ka if len(kb) else torch.zeros_like(ka, dtype=torch.bool)
    return CooTensor(a.rows[hit], a.cols[hit], a.values[hit] * b.values[pos[hit]], a.shape)


def spgemm(a: CooTensor, b: CooTensor) -> CooTensor:
    """Sparse x sparse by expanding every ``a[i, k]`` against row ``k`` of ``b`` (Gustavson), then merging duplicates."""
    bc = b.to_csr()
    cnt = bc.indptr[a.cols + 1] - bc.indptr[a.cols]
    rep = torch.repeat_interleave(torch.arange(len(a.values), device=cnt.device), cnt)
    off = torch.arange(int(cnt.sum()), device=cnt.device) - torch.repeat_interleave(cnt.cumsum(0) - cnt, cnt)
    src = bc.indptr[a.cols][rep] + off
    return CooTensor(a.rows[rep], bc.indices[src], a.values[rep] * bc.values[src], (a.shape[0], b.shape[1])).coalesce()


def sparse_sum(a: CooTensor, dim: int | None = None) -> torch.Tensor:
    if dim is None:
        return a.values.sum()
    idx, n = (a.cols, a.shape[1]) if dim == 0 else (a.rows, a.shape[0])
    return torch.zeros(n, dtype=a.values.dtype).index_add_(0, idx, a.values)


def sparse_norm(a: CooTensor, kind: str = "fro") -> float:
    if kind == "fro":
        return float(a.values.pow(2).sum().sqrt())
    if kind == "1":
        return float(sparse_sum(CooTensor(a.rows, a.cols, a.values.abs(), a.shape), 0).max())
    if kind == "inf":
        return float(sparse_sum(CooTensor(a.rows, a.cols, a.values.abs(), a.shape), 1).max())
    raise ValueError(kind)


def diagonal(a: CooTensor) -> torch.Tensor:
    d = a.rows == a.cols
    return torch.zeros(min(a.shape), dtype=a.values.dtype).index_add_(0, a.rows[d], a.values[d])


def triu(a: CooTensor, k: int = 0): m = a.cols - a.rows >= k; return CooTensor(a.rows[m], a.cols[m], a.values[m], a.shape)
def tril(a: CooTensor, k: int = 0): m = a.cols - a.rows <= k; return CooTensor(a.rows[m], a.cols[m], a.values[m], a.shape)
def identity(n: int, dtype=torch.float64): i = torch.arange(n); return CooTensor(i, i.clone(), torch.ones(n, dtype=dtype), (n, n))


def kron(a: CooTensor, b: CooTensor) -> CooTensor:
    r = (a.rows[:, None] * b.shape[0] + b.rows[None]).reshape(-1)
    c = (a.cols[:, None] * b.shape[1] + b.cols[None]).reshape(-1)
    return CooTensor(r, c, (a.values[:, None] * b.values[None]).reshape(-1), (a.shape[0] * b.shape[0], a.shape[1] * b.shape[1]))


# ================================================================================================ factorisations and solvers
def _rows(csr: CsrTensor):
    ptr, idx, val = csr.indptr.tolist(), csr.indices.tolist(), csr.values.tolist()
    return [dict(zip(idx[ptr[i]:ptr[i + 1]], val[ptr[i]:ptr[i + 1]])) for i in range(csr.shape[0])]


def solve_triangular(t: CooTensor, b: torch.Tensor, lower: bool = True, unit_diagonal: bool = False) -> torch.Tensor:
    rows, x, n = _rows(t.to_csr()), b.double().clone(), t.shape[0]
    for i in (range(n) if lower else range(n - 1, -1, -1)):
        s = x[i] - sum(v * x[j] for j, v in rows[i].items() if (j < i if lower else j > i))
        x[i] = s if unit_diagonal else s / rows[i][i]
    return x


class IncompleteLU:
    """ILU(0): LU restricted to the sparsity pattern of ``A`` (IKJ ordering); ``solve`` applies ``U^-1 L^-1``."""

    def __init__(self, a: CooTensor):
        rows, n = _rows(a.to_csr()), a.shape[0]
        for i in range(n):
            for k in sorted(j for j in rows[i] if j < i):
                if k not in rows[k] or rows[k][k] == 0:
                    continue
                rows[i][k] /= rows[k][k]
                for j, v in rows[k].items():
                    if j > k and j in rows[i]:
                        rows[i][j] -= rows[i][k] * v
        self.rows, self.n = rows, n

    def factors(self) -> tuple[CooTensor, CooTensor]:
        lr, lc, lv, ur, uc, uv = [], [], [], [], [], []
        for i, r in enumerate(self.rows):
            lr.append(i); lc.append(i); lv.append(1.0)
            for j, v in r.items():
                if j < i:
                    lr.append(i); lc.append(j); lv.append(v)
                else:
                    ur.append(i); uc.append(j); uv.append(v)
        t = lambda r, c, v: CooTensor(torch.tensor(r), torch.tensor(c), torch.tensor(v, dtype=torch.float64), (self.n, self.n))
        return t(lr, lc, lv), t(ur, uc, uv)

    def solve(self, b: torch.Tensor) -> torch.Tensor:
        x = b.double().clone()
        for i in range(self.n):
            x[i] -= sum(v * x[j] for j, v in self.rows[i].items() if j < i)
        for i in range(self.n - 1, -1, -1):
            x[i] = (x[i] - sum(v * x[j] for j, v in self.rows[i].items() if j > i)) / self.rows[i][i]
        return x


class SparseCholesky:
    """Up-looking Cholesky of a symmetric positive definite matrix with fill-in (``incomplete=True`` keeps only the pattern
    of the lower triangle of ``A``: IC(0))."""

    def __init__(self, a: CooTensor, incomplete: bool = False):
        n, rows = a.shape[0], _rows(tril(a).to_csr())
        L: list[dict] = [dict() for _ in range(n)]
        for i in range(n):
            cols = sorted(set(rows[i]) - {i}) if incomplete else list(range(i))
            for j in cols:
                s = rows[i].get(j, 0.0) - sum(L[i].get(k, 0.0) * v for k, v in L[j].items() if k < j)
                if s != 0.0 or j in rows[i]:
                    val = s / L[j][j]
                    if val != 0.0:
                        L[i][j] = val
            d = rows[i].get(i, 0.0) - sum(v * v for k, v in L[i].items() if k < i)
            if d <= 0:
                raise ValueError("matrix is not positive definite")
            L[i][i] = math.sqrt(d)
        self.L, self.n = L, n

    def factor(self) -> CooTensor:
        r, c, v = zip(*[(i, j, val) for i, row in enumerate(self.L) for j, val in row.items()])
        return CooTensor(torch.tensor(r), torch.tensor(c), torch.tensor(v, dtype=torch.float64), (self.n, self.n))

    def solve(self, b: torch.Tensor) -> torch.Tensor:
        x = b.double().clone()
        for i in range(self.n):
            x[i] = (x[i] - sum(v * x[j] for j, v in self.L[i].items() if j < i)) / self.L[i][i]
        for i in range(self.n - 1, -1, -1):
            x[i] /= self.L[i][i]
            for j, v in self.L[i].items():
                if j < i:
                    x[j] -= v * x[i]
        return x


def jacobi_preconditioner(a: CooTensor):
    d = diagonal(a).double()
    return lambda r: r / d


def conjugate_gradient(a: CooTensor, b: torch.Tensor, precond=None, tol: float = 1e-10, max_iter: int = 1000, x0=None):
    x = torch.zeros_like(b, dtype=torch.float64) if x0 is None else x0.double().clone()
    M = precond or (lambda r: r)
    r = b.double() - a.matmul(x)
    z = M(r)
    p, rz, bn = z.clone(), r @ z, b.double().norm().clamp(min=1e-300)
    for it in range(max_iter):
        if r.norm() / bn < tol:
            return x, {"iterations": it, "converged": True, "residual": float(r.norm() / bn)}
        ap = a.matmul(p)
        alpha = rz / (p @ ap)
        x, r = x + alpha * p, r - alpha * ap
        z = M(r)
        rz_new = r @ z
        p, rz = z + (rz_new / rz) * p, rz_new
    return x, {"iterations": max_iter, "converged": bool(r.norm() / bn < tol), "residual": float(r.norm() / bn)}


def bicgstab(a: CooTensor, b: torch.Tensor, precond=None, tol: float = 1e-10, max_iter: int = 1000):
    M = precond or (lambda r: r)
    x = torch.zeros_like(b, dtype=torch.float64)
    r = b.double().clone()
    rh, rho, alpha, omega = r.clone(), 1.0, 1.0, 1.0
    v, p, bn = torch.zeros_like(r), torch.zeros_like(r), b.double().norm().clamp(min=1e-300)
    for it in range(max_iter):
        if r.norm() / bn < tol:
            return x, {"iterations": it, "converged": True, "residual": float(r.norm() / bn)}
        rho_new = rh @ r
        p = r + (rho_new / rho) * (alpha / omega) * (p - omega * v)
        ph = M(p)
        v = a.matmul(ph)
        alpha = rho_new / (rh @ v)
        s = r - alpha * v
        sh = M(s)
        t = a.matmul(sh)
        omega = (t @ s) / (t @ t).clamp(min=1e-300)
        x, r, rho = x + alpha * ph + omega * sh, s - omega * t, rho_new
    return x, {"iterations": max_iter, "converged": bool(r.norm() / bn < tol), "residual": float(r.norm() / bn)}


def gmres(a: CooTensor, b: torch.Tensor, precond=None, restart: int = 30, tol: float = 1e-10, max_iter: int = 300):
    """Right-preconditioned restarted GMRES with Givens rotations."""
    M = precond or (lambda r: r)
    b = b.double()
    x, bn, total = torch.zeros_like(b), b.norm().clamp(min=1e-300), 0
    while total < max_iter:
        r = b - a.matmul(x)
        beta = r.norm()
        if beta / bn < tol:
            break
        V, Z = [r / beta], []
        H = torch.zeros(restart + 1, restart, dtype=torch.float64)
        cs, sn, g = [], [], torch.zeros(restart + 1, dtype=torch.float64)
        g[0] = beta
        k_done = 0
        for k in range(restart):
            Z.append(M(V[k]))
            w = a.matmul(Z[k])
            for i in range(k + 1):
                H[i, k] = w @ V[i]
                w = w - H[i, k] * V[i]
            H[k + 1, k] = w.norm()
            for i in range(k):
                H[i, k], H[i + 1, k] = cs[i] * H[i, k] + sn[i] * H[i + 1, k], -sn[i] * H[i, k] + cs[i] * H[i + 1, k]
            den = math.hypot(float(H[k, k]), float(H[k + 1, k]))
            cs.append(float(H[k, k]) / den); sn.append(float(H[k + 1, k]) / den)
            H[k, k], H[k + 1, k] = den, 0.0
            g[k + 1], g[k] = -sn[k] * g[k], cs[k] * g[k]
            total, k_done = total + 1, k + 1
            if abs(float(g[k + 1])) / bn < tol or float(w.norm()) < 1e-14:
                break
            V.append(w / w.norm())
        y = torch.linalg.solve_triangular(H[:k_done, :k_done], g[:k_done, None], upper=True)[:, 0]
        x = x + sum(yi * zi for yi, zi in zip(y, Z))
    res = float((b - a.matmul(x)).norm() / bn)
    return x, {"iterations": total, "converged": res < tol * 10, "residual": res}


def reverse_cuthill_mckee(a: CooTensor) -> torch.Tensor:
    """Bandwidth-reducing permutation: breadth-first levels from a low-degree vertex of every component, neighbours in
    order of degree, result reversed."""
    n = a.shape[0]
    adj: list[set] = [set() for _ in range(n)]
    for i, j in zip(a.rows.tolist(), a.cols.tolist()):
        if i != j:
            adj[i].add(j); adj[j].add(i)
    deg, seen, order = [len(s) for s in adj], [False] * n, []
    for start in sorted(range(n), key=lambda v: deg[v]):
        if seen[start]:
            continue
        seen[start], q = True, deque([start])
        while q:
            v = q.popleft()
            order.append(v)
            for u in sorted(adj[v] - {w for w in adj[v] if seen[w]}, key=lambda w: deg[w]):
                seen[u] = True
                q.append(u)
    return torch.tensor(order[::-1])


def permute(a: CooTensor, perm: torch.Tensor) -> CooTensor:
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(len(perm))
    return CooTensor(inv[a.rows], inv[a.cols], a.values, a.shape)


def bandwidth(a: CooTensor) -> int: return int((a.rows - a.cols).abs().max()) if a.nnz else 0


# ================================================================================================ exchange formats
def write_matrix_market(a: CooTensor, path, symmetric: bool = False, comment: str = "") -> None:
    a = a.coalesce()
    if symmetric:
        a = tril(a)
    kind = "integer" if not a.values.is_floating_point() else "real"
    with open(path, "w") as f:
        f.write(f"%%MatrixMarket matrix coordinate {kind} {'symmetric' if symmetric else 'general'}\n")
        f.writelines(f"%{ln}\n" for ln in comment.splitlines())
        f.write(f"{a.shape[0]} {a.shape[1]} {a.nnz}\n")
        f.writelines(f"{r + 1} {c + 1} {v!r}\n" for r, c, v in zip(a.rows.tolist(), a.cols.tolist(), a.values.tolist()))


def read_matrix_market(path) -> CooTensor:
    """Coordinate format with ``real`` / ``integer`` / ``pattern`` fields and ``general`` / ``symmetric`` / ``skew-symmetric`` symmetry."""
    lines = Path(path).read_text().splitlines()
    head = lines[0].lower().split()
    if head[:3] != ["%%matrixmarket", "matrix", "coordinate"]:
        raise ValueError("only coordinate Matrix Market files are supported")
    field, sym = head[3], head[4]
    body = [ln for ln in lines[1:] if ln.strip() and not ln.startswith("%")]
    m, n, nnz = map(int, body[0].split())
    r, c, v = [], [], []
    for ln in body[1:1 + nnz]:
        p = ln.split()
        r.append(int(p[0]) - 1); c.append(int(p[1]) - 1); v.append(1.0 if field == "pattern" else float(p[2]))
    rows, cols, vals = torch.tensor(r), torch.tensor(c), torch.tensor(v, dtype=torch.float64)
    if sym != "general":
        off = rows != cols
        rows, cols, vals = torch.cat([rows, cols[off]]), torch.cat([cols, rows[off]]), torch.cat([vals, (-1.0 if sym.startswith("skew") else 1.0) * vals[off]])
    return CooTensor(rows, cols, vals, (m, n))


def to_scipy(a, fmt: str = "csr"):
    import scipy.sparse as sps
    coo = a if isinstance(a, CooTensor) else a.to_coo()
    return sps.coo_matrix((coo.values.numpy(), (coo.rows.numpy(), coo.cols.numpy())), shape=coo.shape).asformat(fmt)


def from_scipy(m) -> CooTensor:
    c = m.tocoo()
    return CooTensor(torch.from_numpy(c.row.astype(np.int64)), torch.from_numpy(c.col.astype(np.int64)), torch.from_numpy(c.data.copy()), tuple(c.shape))


def save_matlab(a: CooTensor, path, name: str = "A") -> None:
    from scipy.io import savemat
    savemat(str(path), {name: to_scipy(a, "csc")})


def load_matlab(path, name: str = "A") -> CooTensor:
    from scipy.io import loadmat
    return from_scipy(loadmat(str(path))[name])


# ================================================================================================ analysis and containers
def analyze_pattern(a: CooTensor) -> dict:
    a = a.coalesce()
    m, n = a.shape
    per_row = torch.bincount(a.rows, minlength=m).double()
    offs = (a.cols - a.rows)
    diags = offs.unique()
    key = set((a.rows * n + a.cols).tolist())
    sym = m == n and all((c * n + r) in key for r, c in zip(a.rows.tolist(), a.cols.tolist()))
    bs = next((b for b in (8, 4, 2) if m % b == 0 and n % b == 0 and len(((a.rows // b) * (n // b) + a.cols // b).unique()) * b * b <= 1.5 * a.nnz), 1)
    density = a.nnz / (m * n)
    if len(diags) <= max(5, 0.05 * min(m, n)) and a.nnz >= 0.5 * sum(min(m, n) - abs(int(d)) for d in diags):
        advice = "dia"
    elif bs > 1:
        advice = "bsr"
    elif per_row.max() <= 2 * max(per_row.mean(), 1) and per_row.std() < 0.3 * max(per_row.mean(), 1):
        advice = "ell"
    else:
        advice = "csr" if density < 0.3 else "dense"
    return {"shape": a.shape, "nnz": a.nnz, "density": density, "bandwidth": bandwidth(a), "diagonals": len(diags), "symmetric": bool(sym), "block_size": bs,
            "row_nnz_mean": float(per_row.mean()), "row_nnz_max": int(per_row.max()), "row_nnz_std": float(per_row.std()), "empty_rows": int((per_row == 0).sum()),
            "diagonal_dominant": bool(m == n and (diagonal(a).abs() >= sparse_sum(CooTensor(a.rows, a.cols, a.values.abs(), a.shape), 1) - diagonal(a).abs()).all()),
            "recommended_format": advice}


def memory_report(a: CooTensor, index_bytes: int = 8) -> dict:
    m, n, nnz, vb = a.shape[0], a.shape[1], a.nnz, a.values.element_size()
    per_row = torch.bincount(a.rows, minlength=m)
    out = {"dense": m * n * vb, "coo": nnz * (2 * index_bytes + vb), "csr": (m + 1) * index_bytes + nnz * (index_bytes + vb), "csc": (n + 1) * index_bytes + nnz * (index_bytes + vb),
           "ell": m * int(per_row.max()) * (index_bytes + vb) if nnz else 0}
    out["best"] = min((k for k in out), key=out.get)
    return out


class HybridTensor:
    """ELL part for the first ``k`` entries of every row (``k`` = a quantile of the row lengths) plus a COO part for the
    overflow: regular rows get the fixed-width layout, a few long rows do not inflate it."""

    def __init__(self, a: CooTensor, quantile: float = 0.9):
        a = a.coalesce()
        m = a.shape[0]
        per_row = torch.bincount(a.rows, minlength=m)
        self.k = max(1, int(torch.quantile(per_row.double(), quantile).ceil()))
        start = torch.cat([torch.zeros(1, dtype=torch.long), per_row.cumsum(0)[:-1]])
        rank = torch.arange(a.nnz) - start[a.rows]
        in_ell = rank < self.k
        self.ell_cols = torch.zeros(m, self.k, dtype=torch.long)
        self.ell_vals = torch.zeros(m, self.k, dtype=a.values.dtype)
        self.ell_cols[a.rows[in_ell], rank[in_ell]] = a.cols[in_ell]
        self.ell_vals[a.rows[in_ell], rank[in_ell]] = a.values[in_ell]
        self.coo, self.shape = CooTensor(a.rows[~in_ell], a.cols[~in_ell], a.values[~in_ell], a.shape), a.shape

    def matmul(self, b: torch.Tensor) -> torch.Tensor:
        b2 = b[:, None] if b.dim() == 1 else b
        out = (self.ell_vals[..., None].to(b2.dtype) * b2[self.ell_cols]).sum(1)
        if self.coo.nnz:
            out = out + self.coo.matmul(b2)
        return out[:, 0] if b.dim() == 1 else out

    def to_dense(self):
        d = self.coo.to_dense()
        return d.index_put_((torch.arange(self.shape[0])[:, None].expand_as(self.ell_cols), self.ell_cols), self.ell_vals, accumulate=True)


class SymmetricTensor:
    """Stores the lower triangle only; products use both halves."""

    def __init__(self, a: CooTensor, check: bool = True):
        if check and not torch.allclose(a.to_dense(), a.to_dense().t()):
            raise ValueError("matrix is not symmetric")
        self.lower, self.shape = tril(a.coalesce()), a.shape

    @property
    def nnz_stored(self): return self.lower.nnz

    def matmul(self, b):
        strict = tril(self.lower, -1)
        return self.lower.matmul(b) + strict.transpose().matmul(b)

    def to_coo(self): return sparse_add(self.lower, tril(self.lower, -1).transpose())


# ================================================================================================ layers
class SparseActivation(nn.Module):
    """Applies an activation to the stored values only (zeros stay implicit); valid for functions with ``f(0) = 0``."""

    def __init__(self, kind: str = "relu", negative_slope: float = 0.01):
        super().__init__()
        self.fn = {"relu": torch.relu, "tanh": torch.tanh, "gelu": nn.functional.gelu, "silu": nn.functional.silu, "elu": nn.functional.elu,
                   "leaky_relu": lambda v: nn.functional.leaky_relu(v, negative_slope)}[kind]
        self.prune = kind == "relu"

    def forward(self, a: CooTensor) -> CooTensor:
        v = self.fn(a.values)
        keep = v != 0 if self.prune else torch.ones_like(v, dtype=torch.bool)
        return CooTensor(a.rows[keep], a.cols[keep], v[keep], a.shape)


class SparseLayerNorm(nn.Module):
    """Normalises every row over its stored entries (implicit zeros do not enter the statistics)."""

    def __init__(self, eps: float = 1e-5): super().__init__(); self.eps = eps

    def forward(self, a: CooTensor) -> CooTensor:
        m = a.shape[0]
        cnt = torch.bincount(a.rows, minlength=m).clamp(min=1).to(a.values.dtype)
        mean = torch.zeros(m, dtype=a.values.dtype).index_add_(0, a.rows, a.values) / cnt
        var = torch.zeros(m, dtype=a.values.dtype).index_add_(0, a.rows, (a.values - mean[a.rows]) ** 2) / cnt
        return CooTensor(a.rows, a.cols, (a.values - mean[a.rows]) / torch.sqrt(var[a.rows] + self.eps), a.shape)


def sparse_softmax(a: CooTensor) -> CooTensor:
    """Row softmax over the stored entries."""
    m = a.shape[0]
    mx = torch.full((m,), -math.inf, dtype=a.values.dtype).scatter_reduce(0, a.rows, a.values, "amax")
    e = torch.exp(a.values - mx[a.rows])
    den = torch.zeros(m, dtype=a.values.dtype).index_add_(0, a.rows, e)
    return CooTensor(a.rows, a.cols, e / den[a.rows], a.shape)


class SparseAttention(nn.Module):
    """Attention restricted to a sparse pattern ``(query index, key index)``: scores are computed only at the pattern's
    entries (SDDMM), softmax is over each query's entries, values are gathered by SpMM."""

    def __init__(self, dim: int, heads: int = 1):
        super().__init__()
        self.h, self.q, self.k, self.v, self.o = heads, nn.Linear(dim, dim), nn.Linear(dim, dim), nn.Linear(dim, dim), nn.Linear(dim, dim)

    def forward(self, x: torch.Tensor, rows: torch.Tensor, cols: torch.Tensor) -> torch.Tensor:
        n, d = x.shape
        q, k, v = (f(x).reshape(n, self.h, d // self.h) for f in (self.q, self.k, self.v))
        s = (q[rows] * k[cols]).sum(-1) / math.sqrt(d // self.h)                         # [nnz, heads]
        mx = torch.full((n, self.h), -math.inf, dtype=s.dtype).scatter_reduce(0, rows[:, None].expand_as(s), s, "amax")
        e = torch.exp(s - mx[rows])
        p = e / torch.zeros(n, self.h, dtype=s.dtype).index_add_(0, rows, e)[rows]
        out = torch.zeros(n, self.h, d // self.h, dtype=x.dtype).index_add_(0, rows, p[..., None] * v[cols])
        return self.o(out.reshape(n, d))

    @staticmethod
    def local_pattern(n: int, window: int, global_tokens: int = 0):
        i = torch.arange(n)
        r = i[:, None].expand(n, 2 * window + 1).reshape(-1)
        c = (i[:, None] + torch.arange(-window, window + 1)[None]).reshape(-1)
        ok = (c >= 0) & (c < n)
        r, c = r[ok], c[ok]
        if global_tokens:
            g = torch.arange(global_tokens)
            r = torch.cat([r, i.repeat_interleave(global_tokens), g.repeat_interleave(n)])
            c = torch.cat([c, g.repeat(n), i.repeat(global_tokens)])
            key = (r * n + c).unique()
            r, c = key // n, key % n
        return r, c


class SparseEmbedding(nn.Module):
    """Embedding whose gradient is sparse (rows that were looked up); pairs with the row-wise optimizers below."""

    def __init__(self, num: int, dim: int): super().__init__(); self.inner = nn.Embedding(num, dim, sparse=True)
    def forward(self, idx): return self.inner(idx)


def sparse_max_pool2d(a: torch.Tensor, kernel: int) -> torch.Tensor:
    """Max pooling of a sparse COO ``[H, W]`` torch tensor over its stored entries: windows with no entry stay empty."""
    a = a.coalesce()
    r, c = a.indices()
    key = (r // kernel) * (a.shape[1] // kernel) + c // kernel
    uk, inv = key.unique(return_inverse=True)
    v = torch.full((len(uk),), -math.inf, dtype=a.values().dtype).scatter_reduce(0, inv, a.values(), "amax")
    return torch.sparse_coo_tensor(torch.stack([uk // (a.shape[1] // kernel), uk % (a.shape[1] // kernel)]), v, (a.shape[0] // kernel, a.shape[1] // kernel))


class SparseConv1d(nn.Module):
    """Submanifold-style 1-D convolution on ``(positions, features)``: outputs are produced only at the active input
    positions, from the active neighbours inside the kernel."""

    def __init__(self, cin, cout, kernel_size: int = 3):
        super().__init__()
        self.k, self.weight, self.bias = kernel_size, nn.Parameter(torch.randn(kernel_size, cin, cout) / math.sqrt(cin * kernel_size)), nn.Parameter(torch.zeros(cout))

    def forward(self, pos: torch.Tensor, feats: torch.Tensor):
        order = pos.argsort()
        pos, feats = pos[order], feats[order]
        out = self.bias.expand(len(pos), -1).clone()
        for j in range(self.k):
            want = pos + j - self.k // 2
            at = torch.searchsorted(pos, want).clamp(max=len(pos) - 1)
            hit = pos[at] == want
            out[hit] = out[hit] + feats[at[hit]] @ self.weight[j]
        return pos, out


# ================================================================================================ optimizers
class SparseSGD(torch.optim.Optimizer):
    """SGD with momentum that, for sparse gradients, updates and decays only the rows present in the gradient."""

    def __init__(self, params, lr=0.1, momentum=0.0, weight_decay=0.0): super().__init__(params, dict(lr=lr, momentum=momentum, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self):
        self.rows_touched = 0
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                if p.grad.is_sparse:
                    gr = p.grad.coalesce()
                    idx, val = gr.indices()[0], gr.values()
                    if g["weight_decay"]:
                        val = val + g["weight_decay"] * p[idx]
                    if g["momentum"]:
                        buf = self.state[p].setdefault("momentum", torch.zeros_like(p))
                        buf[idx] = g["momentum"] * buf[idx] + val
                        val = buf[idx]
                    p.index_add_(0, idx, val, alpha=-g["lr"])
                    self.rows_touched += len(idx)
                else:
                    d = p.grad + g["weight_decay"] * p if g["weight_decay"] else p.grad
                    if g["momentum"]:
                        buf = self.state[p].setdefault("momentum", torch.zeros_like(p))
                        buf.mul_(g["momentum"]).add_(d)
                        d = buf
                    p.add_(d, alpha=-g["lr"])


class SparseAdamW(torch.optim.Optimizer):
    """AdamW whose moments, bias correction and decay advance per row, only when that row receives gradient (lazy Adam)."""

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0): super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self):
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["m"], st["v"], st["t"] = torch.zeros_like(p), torch.zeros_like(p), torch.zeros(p.shape[0] if p.dim() else 1)
                if p.grad.is_sparse:
                    gr = p.grad.coalesce()
                    idx, val = gr.indices()[0], gr.values()
                else:
                    idx, val = torch.arange(p.shape[0]), p.grad
                st["t"][idx] += 1
                t = st["t"][idx].reshape(-1, *[1] * (p.dim() - 1))
                st["m"][idx] = b1 * st["m"][idx] + (1 - b1) * val
                st["v"][idx] = b2 * st["v"][idx] + (1 - b2) * val * val
                mh, vh = st["m"][idx] / (1 - b1 ** t), st["v"][idx] / (1 - b2 ** t)
                p[idx] = p[idx] * (1 - g["lr"] * g["weight_decay"]) - g["lr"] * mh / (vh.sqrt() + g["eps"])


class SparseGradientAccumulator:
    """Sums sparse row gradients over micro-batches without ever forming the dense gradient."""

    def __init__(self, shape): self.shape, self.idx, self.val = shape, [], []
    def add(self, grad: torch.Tensor): g = grad.coalesce(); self.idx.append(g.indices()); self.val.append(g.values())
    def result(self) -> torch.Tensor: return torch.sparse_coo_tensor(torch.cat(self.idx, 1), torch.cat(self.val), self.shape).coalesce()
    def clear(self): self.idx, self.val = [], []
