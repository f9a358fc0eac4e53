"""torsh_b200: a Blackwell-native deep-learning framework with ToRSh's API shape.

Facade and prelude in the spirit of ``crates/torsh/src/lib.rs:73-142,438-537``: ``import torsh_b200 as torsh`` gives
``torsh.tensor / zeros / randn``, ``torsh.nn``, ``torsh.optim``, ``torsh.autograd``, ``torsh.data``, ``torsh.distributed``
(alias of :mod:`torsh_b200.parallel`), ``torsh.models``, ``torsh.serialize``."""
__version__ = "0.1.0"

from . import core  # noqa: E402
from .core import DType, Device, DeviceType, RuntimeConfig, Shape, TorshDistributedError, TorshError  # noqa: E402,F401
from . import ops  # noqa: E402,F401
from .ops import attention, elementwise, gemm, linear, multi_tensor, norm, softmax  # noqa: E402,F401
from . import autograd, data, models, nn, optim, parallel, serialize  # noqa: E402,F401
from . import parallel as distributed  # noqa: E402,F401
from . import engine  # noqa: E402,F401
from .tensor import *  # noqa: E402,F401,F403
from .tensor import Tensor  # noqa: E402,F401
from .autograd import enable_grad, no_grad, set_grad_enabled  # noqa: E402,F401
from .serialize import load_tensor, save_tensor  # noqa: E402,F401

float16, bfloat16, float32, float64 = DType.F16, DType.BF16, DType.F32, DType.F64
int8, int16, int32, int64, uint8, bool_ = DType.I8, DType.I16, DType.I32, DType.I64, DType.U8, DType.BOOL


def cuda_is_available() -> bool:
    import torch
    return torch.cuda.is_available()


def device_count() -> int:
    import torch
    return torch.cuda.device_count()


def manual_seed(seed: int):
    import torch
    torch.manual_seed(seed)
