"""``rstorch``: the reference's Python surface (``python/rstorch/__init__.py:19-254``, ``crates/torsh-python/src/lib.rs:
39-80``) served by :mod:`torsh_b200`. Top level: ``Tensor, dtype, device, TorshError, tensor, zeros, ones, randn, rand,
arange, linspace, *_like, empty, full, add/sub/mul/div/matmul/mm/bmm, reshape/view/transpose/permute/squeeze/unsqueeze/
flatten``, dtypes, ``cpu, device_count, is_available, cuda_is_available, mps_is_available, get_device_name, set/get_default_
dtype/device``; sub-modules ``nn, optim, autograd, distributed, data, functional (F)``. In the reference the distributed
functions are stubs returning ``Ok(())`` (``crates/torsh-python/src/distributed.rs:31-204``); here they communicate."""
import torch as _torch

import torsh_b200 as _t
from torsh_b200 import TorshError  # noqa: F401
from torsh_b200.core.device import Device as device, parse_device  # noqa: F401,N813
from torsh_b200.core.dtype import DType as dtype  # noqa: F401,N813
from torsh_b200.tensor import (Tensor, add, arange, bmm, div, empty, empty_like, flatten, full, full_like,  # noqa: F401
                               get_default_device, get_default_dtype, linspace, matmul, mm, mul, ones, ones_like, permute,
                               rand, rand_like, randn, randn_like, reshape, set_default_device, set_default_dtype, squeeze,
                               sub, tensor, transpose, unsqueeze, view, zeros, zeros_like)

from . import autograd, data, distributed, functional, nn, optim  # noqa: E402,F401
from . import functional as F  # noqa: E402,F401,N812

float32, float64, float16, bfloat16 = dtype.F32, dtype.F64, dtype.F16, dtype.BF16
int8, int16, int32, int64, uint8, uint16, uint32, uint64 = dtype.I8, dtype.I16, dtype.I32, dtype.I64, dtype.U8, dtype.U16, dtype.U32, dtype.U64
bool = bool_dtype = dtype.BOOL  # noqa: A001
FloatTensor = DoubleTensor = HalfTensor = LongTensor = IntTensor = ByteTensor = BoolTensor = Tensor  # typed names of the reference all alias Tensor
__version__ = _t.__version__


def cpu():
    return parse_device("cpu")


def device_count():
    return _torch.cuda.device_count()


def is_available():
    return True


def cuda_is_available():
    return _torch.cuda.is_available()


def mps_is_available():
    return False


def get_device_name(index: int = 0):
    return _torch.cuda.get_device_name(index) if _torch.cuda.is_available() else "cpu"
