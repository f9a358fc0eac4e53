"""Run-time generation of fused element-wise CUDA kernels for sm_100a, with measured selection between variants.

An expression over symbolic inputs (``x0 * sigmoid(x1) + 0.5`` ...) is turned into CUDA source: one grid-stride kernel
that reads every input once with 16-byte vector loads, evaluates the whole expression in fp32 registers and writes the
result once. The source is compiled with nvcc for ``sm_100a`` the first time it is needed (cached on disk by content
hash), loaded with ctypes and launched on the caller's stream. Several launch variants (threads per CTA, vectors per
thread) exist per expression; ``KernelSelector`` times them once per size bucket and remembers the winner. On a CPU
tensor the same expression is evaluated with PyTorch ops, so code using it is portable.

The reference has string generators for its backends (crates/torsh-backend/src/kernel_generation/,
``adaptive_kernel_selection.rs``) whose CUDA branch emits a 16x16 SGEMM template and is never compiled; here the
generated code is what runs.
"""
from __future__ import annotations

import ctypes
import hashlib
import math
import os
import threading
from pathlib import Path

import torch

# ---- expression DSL --------------------------------------------------------------------------------------------------
_UNARY = {
    "neg": ("(-{0})", lambda a: -a), "abs": ("fabsf({0})", torch.abs), "exp": ("__expf({0})", torch.exp),
    "log": ("__logf({0})", torch.log), "sqrt": ("sqrtf({0})", torch.sqrt), "rsqrt": ("rsqrtf({0})", torch.rsqrt),
    "tanh": ("tanhf({0})", torch.tanh), "sigmoid": ("(1.f / (1.f + __expf(-{0})))", torch.sigmoid),
    "relu": ("fmaxf({0}, 0.f)", torch.relu), "silu": ("({0} / (1.f + __expf(-{0})))", torch.nn.functional.silu),
    "gelu_tanh": ("(0.5f * {0} * (1.f + tanhf(0.7978845608f * ({0} + 0.044715f * {0} * {0} * {0}))))",
                  lambda a: torch.nn.functional.gelu(a, approximate="tanh")),
    "square": ("({0} * {0})", lambda a: a * a), "reciprocal": ("(1.f / {0})", torch.reciprocal),
}
_BINARY = {
    "add": ("({0} + {1})", torch.add), "sub": ("({0} - {1})", torch.sub), "mul": ("({0} * {1})", torch.mul),
    "div": ("({0} / {1})", torch.div), "max": ("fmaxf({0}, {1})", torch.maximum), "min": ("fminf({0}, {1})", torch.minimum),
    "pow": ("powf({0}, {1})", torch.pow), "gt": ("(({0} > {1}) ? 1.f : 0.f)", lambda a, b: (a > b).to(a.dtype)),
    "lt": ("(({0} < {1}) ? 1.f : 0.f)", lambda a, b: (a < b).to(a.dtype)),
}


class Expr:
    """Node of an element-wise expression. Build with :func:`inputs` and Python operators / the functions below."""

    def __init__(self, op: str, args: tuple = (), value=None):
        self.op, self.args, self.value = op, args, value

    @staticmethod
    def _wrap(v) -> "Expr":
        return v if isinstance(v, Expr) else Expr("const", (), float(v))

    def __add__(self, o): return Expr("add", (self, Expr._wrap(o)))
    def __radd__(self, o): return Expr("add", (Expr._wrap(o), self))
    def __sub__(self, o): return Expr("sub", (self, Expr._wrap(o)))
    def __rsub__(self, o): return Expr("sub", (Expr._wrap(o), self))
    def __mul__(self, o): return Expr("mul", (self, Expr._wrap(o)))
    def __rmul__(self, o): return Expr("mul", (Expr._wrap(o), self))
    def __truediv__(self, o): return Expr("div", (self, Expr._wrap(o)))
    def __rtruediv__(self, o): return Expr("div", (Expr._wrap(o), self))
    def __neg__(self): return Expr("neg", (self,))
    def __pow__(self, o): return Expr("pow", (self, Expr._wrap(o)))

    def key(self) -> str:
        if self.op == "input":
            return f"x{self.value}"
        if self.op == "const":
            return repr(self.value)
        return f"{self.op}({','.join(a.key() for a in self.args)})"

    def n_inputs(self) -> int:
        if self.op == "input":
            return self.value + 1
        return max([a.n_inputs() for a in self.args], default=0)

    def code(self, j: str) -> str:
        """C expression for element ``j`` of the current vectors (inputs are ``f<i>[j]``)."""
        if self.op == "input":
            return f"f{self.value}[{j}]"
        if self.op == "const":
            v = self.value
            if math.isinf(v) or math.isnan(v):
                raise ValueError("constants must be finite")
            return f"{v!r}f" if ("." in repr(v) or "e" in repr(v)) else f"{v!r}.f"
        if self.op == "where":
            c, a, b = (x.code(j) for x in self.args)
            return f"(({c}) != 0.f ? {a} : {b})"
        table = _UNARY if self.op in _UNARY else _BINARY
        return table[self.op][0].format(*(a.code(j) for a in self.args))

    def eval_torch(self, xs):
        if self.op == "input":
            return xs[self.value]
        if self.op == "const":
            return torch.tensor(self.value, dtype=xs[0].dtype, device=xs[0].device)
        if self.op == "where":
            c, a, b = (x.eval_torch(xs) for x in self.args)
            return torch.where(c != 0, a, b)
        table = _UNARY if self.op in _UNARY else _BINARY
        return table[self.op][1](*(a.eval_torch(xs) for a in self.args))


def inputs(n: int) -> list[Expr]:
    return [Expr("input", (), i) for i in range(n)]


def _unary(name):
    return lambda a: Expr(name, (Expr._wrap(a),))


def _binary(name):
    return lambda a, b: Expr(name, (Expr._wrap(a), Expr._wrap(b)))


exp, log, sqrt, rsqrt, tanh, sigmoid, relu, silu, gelu_tanh, square, reciprocal = (
    _unary(n) for n in ("exp", "log", "sqrt", "rsqrt", "tanh", "sigmoid", "relu", "silu", "gelu_tanh", "square", "reciprocal"))
absolute = _unary("abs")
maximum, minimum, greater, less = _binary("max"), _binary("min"), _binary("gt"), _binary("lt")


def where(c, a, b) -> Expr:
    return Expr("where", (Expr._wrap(c), Expr._wrap(a), Expr._wrap(b)))


# ---- source generation -----------------------------------------------------------------------------------------------
_DTYPES = {torch.bfloat16: ("__nv_bfloat16", 8, "__bfloat162float", "__float2bfloat16"), torch.float32: ("float", 4, "", "")}

VARIANTS = {"t256_u1": (256, 1), "t256_u2": (256, 2), "t512_u2": (512, 2), "t128_u4": (128, 4)}   # threads per CTA, vectors in flight per thread


def generate_source(expr: Expr, dtype: torch.dtype) -> str:
    """CUDA source with one kernel template (vectors per thread as parameter) and one ``extern "C"`` launcher per variant."""
    ctype, N, to_f, from_f = _DTYPES[dtype]
    n_in = expr.n_inputs()
    params = ", ".join(f"const {ctype}* __restrict__ in{i}" for i in range(n_in))
    loads = "\n".join(f"        const uint4 r{i} = *reinterpret_cast<const uint4*>(in{i} + v * {N});\n"
                      f"        float f{i}[{N}];\n"
                      f"        {{ const {ctype}* e = reinterpret_cast<const {ctype}*>(&r{i});\n"
                      f"          for (int j = 0; j < {N}; ++j) f{i}[j] = {to_f}(e[j]); }}" for i in range(n_in))
    tail_loads = "\n".join(f"    float f{i}[1] = {{{to_f}(in{i}[i])}};" for i in range(n_in))
    body = expr.code("j")
    tail_body = expr.code("0")
    launchers = []
    for name, (threads, unroll) in VARIANTS.items():
        args = ", ".join(f"(const {ctype}*)ins[{i}]" for i in range(n_in))
        launchers.append(f'''
extern "C" __attribute__((visibility("default"))) int launch_{name}(void** ins, void* out, long n, int device, void* stream) {{
  if (cudaSetDevice(device) != cudaSuccess) return -2;
  if (n <= 0) return 0;
  const long nvec = n / {N};
  long grid = (nvec + {threads * unroll - 1}L) / {threads * unroll};
  if (grid < 1) grid = 1;
  if (grid > 148L * 16) grid = 148L * 16;
  fused_kernel<{unroll}><<<(unsigned)grid, {threads}, 0, (cudaStream_t)stream>>>({args}, ({ctype}*)out, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}}''')
    return f'''// generated by torsh_b200.core.kernel_gen for: {expr.key()}
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

template <int UNROLL>
__global__ void fused_kernel({params}, {ctype}* __restrict__ out, long n) {{
  const long nvec = n / {N};
  const long stride = (long)gridDim.x * blockDim.x;
  for (long v0 = (long)blockIdx.x * blockDim.x + threadIdx.x; v0 < nvec; v0 += stride * UNROLL) {{
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {{
      const long v = v0 + u * stride;
      if (v < nvec) {{
{loads}
        uint4 o;
        {ctype}* oe = reinterpret_cast<{ctype}*>(&o);
#pragma unroll
        for (int j = 0; j < {N}; ++j) oe[j] = {from_f}({body});
        *reinterpret_cast<uint4*>(out + v * {N}) = o;
      }}
    }}
  }}
  // elements past the last full vector
  for (long i = nvec * {N} + (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {{
{tail_loads}
    out[i] = {from_f}({tail_body});
  }}
}}
{"".join(launchers)}
'''


def jit_directory() -> Path:
    d = Path(os.environ.get("TORSH_JIT_DIR") or (Path.home() / ".cache" / "torsh_b200" / "jit"))
    d.mkdir(parents=True, exist_ok=True)
    return d


def compile_source(source: str, name: str | None = None) -> Path:
    """nvcc for sm_100a into the JIT directory (content-addressed: an unchanged source is not rebuilt)."""
    from ..utils import cpp_extension as ce
    h = hashlib.sha256(source.encode()).hexdigest()[:16]
    name = name or f"tbjit_{h}"
    src = jit_directory() / f"{name}.cu"
    if not src.exists() or src.read_text() != source:
        src.write_text(source)
    return ce.build(ce.CppExtensionConfig(name, [str(src)], extra_cuda_cflags=["-O3", "-lineinfo", "--use_fast_math"],
                                          build_directory=str(jit_directory())))


# ---- measured selection ----------------------------------------------------------------------------------------------
class KernelSelector:
    """Chooses a launch variant per (kernel, size bucket) by timing each once (CUDA events) and remembering the winner;
    the table can be saved and reloaded, so production runs need not tune."""

    def __init__(self, path: str | None = None):
        from .backend import Autotuner
        self.tuner = Autotuner(path, warmup=2, iters=5)

    @staticmethod
    def bucket(n: int) -> int:
        return max(int(math.log2(max(n, 1))), 10)

    def choose(self, kernel_key: str, n: int, run_variant) -> str:
        """``run_variant(name)`` launches the kernel once with that variant."""
        key = f"{kernel_key}|2^{self.bucket(n)}"
        return self.tuner.select(key, {name: (lambda name=name: run_variant(name)) for name in VARIANTS})


_selector = None
_lock = threading.Lock()


def default_selector() -> KernelSelector:
    global _selector
    with _lock:
        if _selector is None:
            _selector = KernelSelector(os.environ.get("TORSH_KERNEL_TUNE_FILE"))
        return _selector


class FusedElementwise:
    """Callable built from ``fn(*inputs) -> Expr``. bf16 / fp32 CUDA tensors of equal shape run the generated kernel; other
    tensors evaluate the same expression with PyTorch ops."""

    def __init__(self, fn, n_inputs: int, tune: bool = True):
        self.expr = Expr._wrap(fn(*inputs(n_inputs)))
        self.n_inputs = n_inputs
        self.tune = tune
        self._libs: dict = {}

    def source(self, dtype: torch.dtype = torch.bfloat16) -> str:
        return generate_source(self.expr, dtype)

    def _lib(self, dtype):
        lib = self._libs.get(dtype)
        if lib is None:
            lib = ctypes.CDLL(str(compile_source(self.source(dtype))), mode=ctypes.RTLD_LOCAL)
            for name in VARIANTS:
                f = getattr(lib, f"launch_{name}")
                f.restype = ctypes.c_int
                f.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p, ctypes.c_long, ctypes.c_int, ctypes.c_void_p]
            self._libs[dtype] = lib
        return lib

    def __call__(self, *xs: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        if len(xs) != self.n_inputs:
            raise ValueError(f"expected {self.n_inputs} inputs")
        x0 = xs[0]
        ok = (x0.is_cuda and x0.dtype in _DTYPES and all(x.shape == x0.shape and x.dtype == x0.dtype and x.is_cuda for x in xs))
        if not ok:
            r = self.expr.eval_torch([x.float() for x in xs]).to(x0.dtype)
            if out is not None:
                out.copy_(r)
                return out
            return r
        xs = [x.contiguous() for x in xs]
        out = torch.empty_like(xs[0]) if out is None else out
        if any(x.data_ptr() % 16 for x in xs) or out.data_ptr() % 16:
            out.copy_(self.expr.eval_torch([x.float() for x in xs]).to(x0.dtype))
            return out
        lib = self._lib(x0.dtype)
        ptrs = (ctypes.c_void_p * self.n_inputs)(*[x.data_ptr() for x in xs])
        n, dev = xs[0].numel(), x0.device.index or 0
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

        def run(name):
            rc = getattr(lib, f"launch_{name}")(ptrs, out.data_ptr(), n, dev, stream)
            if rc != 0:
                raise RuntimeError(f"generated kernel launch failed (variant {name}, rc {rc})")
        variant = default_selector().choose(f"{self.expr.key()}|{x0.dtype}", n, run) if self.tune else "t256_u2"
        run(variant)
        return out
