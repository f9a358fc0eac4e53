"""Tensor creation and the ``Tensor`` handle (``crates/torsh-tensor/src/creation.rs``, ``src/lib.rs:168-195``).

``Tensor`` is ``torch.Tensor``: device-resident, strided, differentiable. The reference's tensors are host ``Vec<T>``
with a device tag (``crates/torsh-tensor/src/core_ops/types.rs:22-44``); its ``tensor!`` / ``tensor_2d!`` macros map to
:func:`tensor` / :func:`tensor_2d`. Device-resident elementwise / reduction entry points route CUDA bf16/fp32 tensors
to this package's kernels (see :mod:`torsh_b200.ops.elementwise`)."""
from __future__ import annotations

import torch

from .core.device import parse_device
from .core.dtype import to_torch_dtype
from .ops import elementwise as _ew

Tensor = torch.Tensor
_default_device = torch.device("cpu")


def set_default_device(dev):
    global _default_device
    _default_device = parse_device(dev).torch()


def get_default_device():
    return _default_device


def set_default_dtype(dt):
    torch.set_default_dtype(to_torch_dtype(dt))


def get_default_dtype():
    return torch.get_default_dtype()


def _kw(dtype, device, requires_grad=False):
    kw = {"device": parse_device(device).torch() if device is not None else _default_device, "requires_grad": requires_grad}
    if dtype is not None:
        kw["dtype"] = to_torch_dtype(dtype)
    return kw


def tensor(data, dtype=None, device=None, requires_grad=False): return torch.tensor(data, **_kw(dtype, device, requires_grad))
def tensor_2d(rows, dtype=None, device=None): return torch.tensor([list(r) for r in rows], **_kw(dtype, device))
def zeros(*shape, dtype=None, device=None, requires_grad=False): return torch.zeros(*shape, **_kw(dtype, device, requires_grad))
def ones(*shape, dtype=None, device=None, requires_grad=False): return torch.ones(*shape, **_kw(dtype, device, requires_grad))
def empty(*shape, dtype=None, device=None): return torch.empty(*shape, **_kw(dtype, device))
def full(shape, value, dtype=None, device=None): return torch.full(tuple(shape), value, **_kw(dtype, device))
def rand(*shape, dtype=None, device=None, requires_grad=False): return torch.rand(*shape, **_kw(dtype, device, requires_grad))
def randn(*shape, dtype=None, device=None, requires_grad=False): return torch.randn(*shape, **_kw(dtype, device, requires_grad))
def eye(n, m=None, dtype=None, device=None): return torch.eye(n, m if m is not None else n, **_kw(dtype, device))
def arange(*a, dtype=None, device=None): return torch.arange(*a, **_kw(dtype, device))
def linspace(start, end, steps, dtype=None, device=None): return torch.linspace(start, end, steps, **_kw(dtype, device))
zeros_like, ones_like, rand_like, randn_like, empty_like, full_like = (torch.zeros_like, torch.ones_like, torch.rand_like,
                                                                       torch.randn_like, torch.empty_like, torch.full_like)


def from_numpy(a):
    return torch.from_numpy(a)


# ---- math entry points (kernels on CUDA bf16/fp32, PyTorch otherwise) ------------------------------------
def add(a, b): return _ew.binary("add", a, b)
def sub(a, b): return _ew.binary("sub", a, b)
def mul(a, b): return _ew.binary("mul", a, b)
def div(a, b): return _ew.binary("div", a, b)
def maximum(a, b): return _ew.binary("max", a, b)
def minimum(a, b): return _ew.binary("min", a, b)
def exp(x): return _ew.unary("exp", x)
def log(x): return _ew.unary("log", x)
def sqrt(x): return _ew.unary("sqrt", x)
def abs(x): return _ew.unary("abs", x)  # noqa: A001
def neg(x): return _ew.unary("neg", x)
relu, sigmoid, tanh, gelu, silu = _ew.relu, _ew.sigmoid, _ew.tanh, _ew.gelu, _ew.silu
def sum(x, dim=None, keepdim=False): return x.sum() if dim is None else _ew.reduce("sum", x, dim, keepdim)  # noqa: A001
def mean(x, dim=None, keepdim=False): return x.mean() if dim is None else _ew.reduce("mean", x, dim, keepdim)
def max(x, dim=None, keepdim=False): return x.max() if dim is None else _ew.reduce("max", x, dim, keepdim)  # noqa: A001
def min(x, dim=None, keepdim=False): return x.min() if dim is None else _ew.reduce("min", x, dim, keepdim)  # noqa: A001


def matmul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """2-D bf16 CUDA operands run the tcgen05 GEMM (``b`` is ``[K, N]``, consumed MN-major: no transpose copy)."""
    if (a.is_cuda and a.dim() == 2 and b.dim() == 2 and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
            and a.shape[1] % 8 == 0 and b.shape[1] % 8 == 0 and a.is_contiguous() and b.is_contiguous()
            and not (torch.is_grad_enabled() and (a.requires_grad or b.requires_grad))):
        from .ops.gemm import gemm
        return gemm(a, b, b_major=1)
    return torch.matmul(a, b)


mm, bmm = matmul, torch.bmm
reshape, view, transpose, permute = torch.reshape, lambda t, *s: t.view(*s), torch.transpose, torch.permute
squeeze, unsqueeze, flatten, cat, stack = torch.squeeze, torch.unsqueeze, torch.flatten, torch.cat, torch.stack
softmax, log_softmax = lambda x, dim=-1: __import__("torsh_b200").ops.softmax.softmax(x, dim), \
    lambda x, dim=-1: __import__("torsh_b200").ops.softmax.log_softmax(x, dim)
