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


def test_reference_named_surface_is_complete_and_correct():
    """Every function name the reference exports from its C layer resolves here, and the ones this file had not touched
    yet compute what their names say."""
    import json
    import torch
    lib = _lib()
    P = ctypes.c_void_p
    names = """adam_create clear_last_error cuda_device_memory cuda_device_name get_device_id get_device_type get_memory_usage
        get_num_threads get_peak_memory_usage has_error is_autocast_enabled is_debug_mode_enabled linear_create
        linear_get_input_features linear_get_output_features module_free reset_memory_tracking set_autocast set_debug_mode
        set_num_threads sgd_create sgd_step start_profiling stop_profiling tensor_adam_step_inplace tensor_axpy_inplace
        tensor_div_scalar tensor_eye tensor_linspace tensor_max_dim tensor_min_dim tensor_multiply tensor_scalar tensor_size
        tensor_sub_scalar tensor_tan""".split()
    for n in names:
        assert hasattr(lib, "torsh_" + n), n
    for n in ("tensor_eye", "tensor_linspace", "tensor_scalar", "tensor_sub_scalar", "tensor_div_scalar", "tensor_tan",
              "tensor_max_dim", "tensor_min_dim", "linear_create", "sgd_create", "adam_create"):
        getattr(lib, "torsh_" + n).restype = P
    for n in ("tensor_size", "get_memory_usage", "get_peak_memory_usage", "linear_get_input_features", "linear_get_output_features"):
        getattr(lib, "torsh_" + n).restype = ctypes.c_size_t
    lib.torsh_stop_profiling.restype = ctypes.c_char_p
    lib.torsh_tensor_linspace.argtypes = [ctypes.c_double, ctypes.c_double, ctypes.c_size_t]
    lib.torsh_tensor_max_dim.argtypes = lib.torsh_tensor_min_dim.argtypes = [P, ctypes.c_int]
    lib.torsh_tensor_sub_scalar.argtypes = lib.torsh_tensor_div_scalar.argtypes = [P, ctypes.c_float]
    lib.torsh_tensor_scalar.argtypes = [ctypes.c_float]
    lib.torsh_tensor_eye.argtypes = [ctypes.c_size_t]
    lib.torsh_tensor_axpy_inplace.argtypes = [P, P, ctypes.c_float]
    lib.torsh_tensor_adam_step_inplace.argtypes = [P, P, P, P] + [ctypes.c_float] * 4 + [ctypes.c_int64]
    lib.torsh_linear_create.argtypes = [ctypes.c_size_t, ctypes.c_size_t, ctypes.c_bool]
    lib.torsh_sgd_create.argtypes = [ctypes.c_float]
    lib.torsh_adam_create.argtypes = [ctypes.c_float] * 4

    lib.torsh_reset_memory_tracking()
    before = lib.torsh_get_memory_usage()
    assert lib.torsh_start_profiling() == 0
    eye = P(lib.torsh_tensor_eye(4))
    assert np.array_equal(_np(lib, eye, (4, 4)), np.eye(4, dtype=np.float32)) and lib.torsh_tensor_size(eye) == 16
    assert lib.torsh_get_memory_usage() >= before + 64 and lib.torsh_get_peak_memory_usage() >= lib.torsh_get_memory_usage()
    ls = P(lib.torsh_tensor_linspace(0.0, 1.0, 5))
    assert np.allclose(_np(lib, ls, (5,)), np.linspace(0, 1, 5))
    a = np.arange(12, dtype=np.float32).reshape(3, 4) / 7 - 0.5
    ta = _mk(lib, a)
    assert np.allclose(_np(lib, P(lib.torsh_tensor_sub_scalar(ta, 0.25)), (3, 4)), a - 0.25)
    assert np.allclose(_np(lib, P(lib.torsh_tensor_div_scalar(ta, 4.0)), (3, 4)), a / 4)
    assert np.allclose(_np(lib, P(lib.torsh_tensor_tan(ta)), (3, 4)), np.tan(a), atol=1e-6)
    assert np.allclose(_np(lib, P(lib.torsh_tensor_max_dim(ta, 1)), (3,)), a.max(1))
    assert np.allclose(_np(lib, P(lib.torsh_tensor_min_dim(ta, 0)), (4,)), a.min(0))
    assert _np(lib, P(lib.torsh_tensor_scalar(2.5)), ())[()] == 2.5
    out = _mk(lib, np.zeros_like(a))
    assert lib.torsh_tensor_multiply(ta, ta, out) == 0 and np.allclose(_np(lib, out, (3, 4)), a * a)
    assert lib.torsh_tensor_axpy_inplace(out, ta, 2.0) == 0 and np.allclose(_np(lib, out, (3, 4)), a * a + 2 * a)
    # explicit Adam steps against torch.optim.Adam
    w0 = np.linspace(-1, 1, 8, dtype=np.float32)
    p = torch.nn.Parameter(torch.from_numpy(w0.copy()))
    opt = torch.optim.Adam([p], lr=0.1, betas=(0.9, 0.99), eps=1e-8)
    tp, tm, tv = _mk(lib, w0), _mk(lib, np.zeros(8)), _mk(lib, np.zeros(8))
    for step in range(1, 4):
        g = (np.cos(np.arange(8)) * step).astype(np.float32)
        p.grad = torch.from_numpy(g.copy())
        opt.step()
        assert lib.torsh_tensor_adam_step_inplace(tp, _mk(lib, g), tm, tv, 0.1, 0.9, 0.99, 1e-8, step) == 0
    assert np.allclose(_np(lib, tp, (8,)), p.detach().numpy(), atol=1e-6)
    # reference-named layer / optimizer constructors drive the same objects
    lin = P(lib.torsh_linear_create(3, 2, True))
    assert lib.torsh_linear_get_input_features(lin) == 3 and lib.torsh_linear_get_output_features(lin) == 2
    sgd = P(lib.torsh_sgd_create(0.5))
    assert lib.torsh_optimizer_add_linear(sgd, lin) == 0
    w_before = _np(lib, P(lib.torsh_linear_weight(lin)), (3, 2))
    x = _mk(lib, np.ones((1, 3)))
    lib.torsh_tensor_free(P(lib.torsh_linear_forward(lin, x)))
    lib.torsh_tensor_free(P(lib.torsh_linear_backward(lin, _mk(lib, np.ones((1, 2))))))
    assert lib.torsh_sgd_step(sgd) == 0
    assert np.allclose(_np(lib, P(lib.torsh_linear_weight(lin)), (3, 2)), w_before - 0.5)
    adam = P(lib.torsh_adam_create(0.1, 0.9, 0.999, 1e-8))
    assert lib.torsh_sgd_step(adam) != 0 and lib.torsh_has_error() == 1
    lib.torsh_clear_last_error()
    assert lib.torsh_has_error() == 0
    # settings
    assert lib.torsh_set_num_threads(4) == 0 and lib.torsh_get_num_threads() == 4 and lib.torsh_set_num_threads(0) != 0
    assert lib.torsh_set_autocast(1) == 0 and lib.torsh_is_autocast_enabled() == 1
    assert lib.torsh_set_debug_mode(1) == 0 and lib.torsh_is_debug_mode_enabled() == 1
    lib.torsh_set_autocast(0); lib.torsh_set_debug_mode(0)
    assert lib.torsh_get_device_type() == 0 and lib.torsh_get_device_id() == 0
    prof = json.loads(lib.torsh_stop_profiling().decode())
    assert prof["elapsed_ms"] > 0 and prof["peak_memory_bytes"] >= prof["memory_bytes"] > 0
    lib.torsh_module_free(lin); lib.torsh_optimizer_free(sgd); lib.torsh_optimizer_free(adam)
