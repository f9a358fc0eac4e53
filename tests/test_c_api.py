"""The C ABI (csrc/include/torsh.h) exercised through ctypes the way a foreign-language binding would."""
import ctypes

import numpy as np


def _lib():
    from torsh_b200 import _native as nv
    lib = nv.host()
    P, I64 = ctypes.c_void_p, ctypes.c_int64
    for name in ("tensor_new", "tensor_zeros", "tensor_ones", "tensor_randn", "tensor_add", "tensor_mul", "tensor_matmul",
                 "tensor_relu", "tensor_softmax", "tensor_sum_dim", "tensor_transpose", "tensor_conv2d", "tensor_mean_all",
                 "linear_new", "linear_forward", "linear_backward", "linear_weight", "sgd_new", "adam_new"):
        getattr(lib, "torsh_" + name).restype = P
    lib.torsh_tensor_data.restype = ctypes.POINTER(ctypes.c_float)
    lib.torsh_tensor_numel.restype = I64
    lib.torsh_get_last_error.restype = ctypes.c_char_p
    lib.torsh_version.restype = ctypes.c_char_p
    return lib


def _mk(lib, arr):
    arr = np.ascontiguousarray(arr, dtype=np.float32)
    shape = (ctypes.c_int64 * arr.ndim)(*arr.shape)
    return ctypes.c_void_p(lib.torsh_tensor_new(arr.ctypes.data_as(ctypes.c_void_p), shape, arr.ndim))


def _np(lib, t, shape):
    n = lib.torsh_tensor_numel(t)
    return np.ctypeslib.as_array(lib.torsh_tensor_data(t), shape=(n,)).reshape(shape).copy()


def test_tensor_ops_match_numpy():
    lib = _lib()
    assert lib.torsh_init() == 0 and lib.torsh_version() == b"0.1.0"
    rng = np.random.default_rng(0)
    a, b = rng.standard_normal((3, 4)).astype(np.float32), rng.standard_normal((4, 5)).astype(np.float32)
    ta, tb = _mk(lib, a), _mk(lib, b)
    c = ctypes.c_void_p(lib.torsh_tensor_matmul(ta, tb))
    assert np.allclose(_np(lib, c, (3, 5)), a @ b, atol=1e-5)
    s = ctypes.c_void_p(lib.torsh_tensor_softmax(ta, ctypes.c_int(1)))
    e = np.exp(a - a.max(1, keepdims=True))
    assert np.allclose(_np(lib, s, (3, 4)), e / e.sum(1, keepdims=True), atol=1e-6)
    t = ctypes.c_void_p(lib.torsh_tensor_transpose(ta, 0, 1))
    assert np.allclose(_np(lib, t, (4, 3)), a.T)
    assert lib.torsh_tensor_matmul(ta, ta) is None and b"mismatch" in lib.torsh_get_last_error()
    x = rng.standard_normal((1, 2, 5, 5)).astype(np.float32)
    w = rng.standard_normal((3, 2, 3, 3)).astype(np.float32)
    y = ctypes.c_void_p(lib.torsh_tensor_conv2d(_mk(lib, x), _mk(lib, w), None, 1, 1))
    import torch
    ref = torch.nn.functional.conv2d(torch.from_numpy(x), torch.from_numpy(w), padding=1).numpy()
    assert np.allclose(_np(lib, y, ref.shape), ref, atol=1e-4)


def test_linear_training_through_c_api():
    lib = _lib()
    lib.torsh_set_random_seed(ctypes.c_uint64(1))
    lin = ctypes.c_void_p(lib.torsh_linear_new(ctypes.c_int64(3), ctypes.c_int64(1), 1))
    opt = ctypes.c_void_p(lib.torsh_adam_new(ctypes.c_float(0.05), ctypes.c_float(0.9), ctypes.c_float(0.999),
                                             ctypes.c_float(1e-8), ctypes.c_float(0.0), 1))
    assert lib.torsh_optimizer_add_linear(opt, lin) == 0
    rng = np.random.default_rng(1)
    X = rng.standard_normal((64, 3)).astype(np.float32)
    Y = (X @ np.array([[1.0], [-2.0], [0.5]], dtype=np.float32) + 0.3).astype(np.float32)
    tx = _mk(lib, X)
    first = last = None
    for _ in range(300):
        pred = ctypes.c_void_p(lib.torsh_linear_forward(lin, tx))
        p = _np(lib, pred, (64, 1))
        loss = float(((p - Y) ** 2).mean())
        first = loss if first is None else first
        last = loss
        g = _mk(lib, 2 * (p - Y) / 64)
        lib.torsh_optimizer_zero_grad(opt)
        gx = lib.torsh_linear_backward(lin, g)
        lib.torsh_tensor_free(ctypes.c_void_p(gx)); lib.torsh_tensor_free(g); lib.torsh_tensor_free(pred)
        lib.torsh_optimizer_step(opt)
    assert last < 0.01 * first
