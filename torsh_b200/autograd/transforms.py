"""Differentiable-programming tools on top of PyTorch autograd: functional transforms (grad, value_and_grad, vmap, jvp,
vjp, jacfwd, jacrev, hessian), higher-order and meta-gradients, implicit differentiation (fixed points, argmin of an inner
problem), ODE integration with gradients (RK4 / adaptive Dormand-Prince), surrogate gradients for discrete operations
(straight-through, Gumbel-softmax) and score-function estimators for stochastic nodes, symbolic differentiation of small
expressions, gradient-flow analysis and filtering, staleness compensation for delayed gradients, hypergradient descent for
the learning rate, DARTS-style mixed operations and a DOT rendering of the autograd graph.

Reference modules: crates/torsh-autograd/src/{jax_transformations,higher_order_gradients,meta_gradient,iterative_solvers,
optimization_diff,neural_ode,discrete_ops,stochastic_graphs,symbolic,gradient_flow_analysis,gradient_filtering,
staleness_handling,hyperparameter_optimization,neural_architecture_search,graph_visualization}.rs.
"""
from __future__ import annotations

import math
from collections import deque
from dataclasses import dataclass

import torch
from torch import nn

# ---- functional transforms -------------------------------------------------------------------------------------------
grad = torch.func.grad
vmap = torch.func.vmap
jvp = torch.func.jvp
vjp = torch.func.vjp
jacfwd = torch.func.jacfwd
jacrev = torch.func.jacrev
hessian = torch.func.hessian


def value_and_grad(fn, argnums=0, has_aux: bool = False):
    """``f(*args) -> (value, gradient)`` in JAX's order (torch.func returns the gradient first)."""
    gv = torch.func.grad_and_value(fn, argnums=argnums, has_aux=has_aux)
    return lambda *a, **k: tuple(reversed(gv(*a, **k)))


def nth_derivative(fn, n: int):
    """Scalar function -> its n-th derivative."""
    for _ in range(n):
        fn = torch.func.grad(fn)
    return fn


def hessian_vector_product(fn, x: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """H(x) v by forward-over-reverse differentiation (no Hessian is formed)."""
    return torch.func.jvp(torch.func.grad(fn), (x,), (v,))[1]


# ---- meta-gradients --------------------------------------------------------------------------------------------------
def unrolled_meta_gradient(inner_loss, outer_loss, params: dict, meta_params, inner_lr: float, steps: int = 1):
    """d outer_loss(theta_K) / d meta_params where theta_k+1 = theta_k - lr * d inner_loss(theta_k, meta) / d theta (the
    inner updates stay in the graph)."""
    theta = dict(params)
    for _ in range(steps):
        l = inner_loss(theta, meta_params)
        g = torch.autograd.grad(l, list(theta.values()), create_graph=True)
        theta = {k: p - inner_lr * gi for (k, p), gi in zip(theta.items(), g)}
    out = outer_loss(theta, meta_params)
    metas = list(meta_params.values()) if isinstance(meta_params, dict) else list(meta_params)
    return out, torch.autograd.grad(out, metas, allow_unused=True)


# ---- implicit differentiation ------------------------------------------------------------------------------------------
class _FixedPoint(torch.autograd.Function):
    @staticmethod
    def forward(ctx, f, x0, tol, max_iter, *params):
        with torch.no_grad():
            z = x0
            for _ in range(max_iter):
                z_new = f(z, *params)
                if (z_new - z).norm() <= tol * (1 + z.norm()):
                    z = z_new
                    break
                z = z_new
        ctx.f, ctx.tol, ctx.max_iter = f, tol, max_iter
        ctx.save_for_backward(z, *params)
        return z

    @staticmethod
    def backward(ctx, gz):
        z, *params = ctx.saved_tensors
        with torch.enable_grad():
            zd = z.detach().requires_grad_(True)
            pd = [p.detach().requires_grad_(p.requires_grad) for p in params]
            fz = ctx.f(zd, *pd)
        # solve u = gz + J_z^T u by the same kind of iteration (the adjoint fixed point)
        u = gz.clone()
        for _ in range(ctx.max_iter):
            un = gz + torch.autograd.grad(fz, zd, u, retain_graph=True)[0]
            if (un - u).norm() <= ctx.tol * (1 + u.norm()):
                u = un
                break
            u = un
        need = [p for p in pd if p.requires_grad]
        gp = torch.autograd.grad(fz, need, u, allow_unused=True) if need else ()
        it = iter(gp)
        return (None, None, None, None, *[next(it) if p.requires_grad else None for p in pd])


def fixed_point(f, x0: torch.Tensor, *params, tol: float = 1e-6, max_iter: int = 200) -> torch.Tensor:
    """z* with z* = f(z*, *params); gradients w.r.t. ``params`` by the implicit function theorem (no unrolling stored)."""
    return _FixedPoint.apply(f, x0, tol, max_iter, *params)


def argmin_implicit_gradient(inner_loss, x_star: torch.Tensor, theta: torch.Tensor, outer_grad_x: torch.Tensor) -> torch.Tensor:
    """d L_outer / d theta through x*(theta) = argmin_x inner_loss(x, theta):  - (d^2 f / d theta dx) (d^2 f / dx^2)^-1 g_x."""
    x = x_star.detach().requires_grad_(True)
    th = theta.detach().requires_grad_(True)
    gx = torch.autograd.grad(inner_loss(x, th), x, create_graph=True)[0]
    H = torch.stack([torch.autograd.grad(gx.reshape(-1)[i], x, retain_graph=True)[0].reshape(-1) for i in range(x.numel())])
    v = torch.linalg.solve(H, outer_grad_x.reshape(-1))
    return -torch.autograd.grad(gx.reshape(-1), th, v)[0]


# ---- ODE integration ---------------------------------------------------------------------------------------------------
def odeint(f, y0: torch.Tensor, t: torch.Tensor, method: str = "rk4", rtol: float = 1e-5, atol: float = 1e-7, steps_per_interval: int = 8):
    """Solution of dy/dt = f(t, y) at the times ``t`` (``[T, ...]``). ``rk4`` uses fixed sub-steps; ``dopri5`` adapts its
    step to the tolerances. Every arithmetic step is differentiable, so gradients flow to ``y0`` and to parameters used in ``f``."""
    ys, y = [y0], y0
    for t0, t1 in zip(t[:-1], t[1:]):
        if method == "rk4":
            h = (t1 - t0) / steps_per_interval
            tt = t0
            for _ in range(steps_per_interval):
                k1 = f(tt, y)
                k2 = f(tt + h / 2, y + h / 2 * k1)
                k3 = f(tt + h / 2, y + h / 2 * k2)
                k4 = f(tt + h, y + h * k3)
                y = y + h / 6 * (k1 + 2 * k2 + 2 * k3 + k4)
                tt = tt + h
        elif method == "dopri5":
            y = _dopri5_interval(f, y, t0, t1, rtol, atol)
        else:
            raise ValueError(f"unknown method {method!r}")
        ys.append(y)
    return torch.stack(ys)


_DP_C = [0, 1 / 5, 3 / 10, 4 / 5, 8 / 9, 1, 1]
_DP_A = [[], [1 / 5], [3 / 40, 9 / 40], [44 / 45, -56 / 15, 32 / 9], [19372 / 6561, -25360 / 2187, 64448 / 6561, -212 / 729],
         [9017 / 3168, -355 / 33, 46732 / 5247, 49 / 176, -5103 / 18656], [35 / 384, 0, 500 / 1113, 125 / 192, -2187 / 6784, 11 / 84]]
_DP_B5 = [35 / 384, 0, 500 / 1113, 125 / 192, -2187 / 6784, 11 / 84, 0]
_DP_B4 = [5179 / 57600, 0, 7571 / 16695, 393 / 640, -92097 / 339200, 187 / 2100, 1 / 40]


def _dopri5_interval(f, y, t0, t1, rtol, atol):
    t, h = t0, (t1 - t0) / 4
    for _ in range(10000):
        if float(t1 - t) <= 1e-12 * max(1.0, abs(float(t1))):
            break
        h = torch.minimum(h, t1 - t) if isinstance(h, torch.Tensor) else min(h, t1 - t)
        ks = []
        for i in range(7):
            yi = y + h * sum(a * k for a, k in zip(_DP_A[i], ks)) if i else y
            ks.append(f(t + _DP_C[i] * h, yi))
        y5 = y + h * sum(b * k for b, k in zip(_DP_B5, ks))
        y4 = y + h * sum(b * k for b, k in zip(_DP_B4, ks))
        with torch.no_grad():
            scale = atol + rtol * torch.maximum(y.abs(), y5.abs())
            err = float(((y5 - y4) / scale).pow(2).mean().sqrt())
        if err <= 1.0:
            t, y = t + h, y5
        with torch.no_grad():
            h = h * min(5.0, max(0.2, 0.9 * (1.0 / max(err, 1e-10)) ** 0.2))
    return y


# ---- discrete operations and stochastic nodes --------------------------------------------------------------------------
class _StraightThrough(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, fn):
        return fn(x)

    @staticmethod
    def backward(ctx, g):
        return g, None


def straight_through(x: torch.Tensor, fn=torch.round) -> torch.Tensor:
    """``fn(x)`` forward (round, sign, argmax one-hot ...), identity gradient backward."""
    return _StraightThrough.apply(x, fn)


def gumbel_softmax(logits: torch.Tensor, tau: float = 1.0, hard: bool = False, generator=None) -> torch.Tensor:
    u = torch.rand(logits.shape, generator=generator, device=logits.device).clamp(1e-10, 1 - 1e-10)
    y = torch.softmax((logits - torch.log(-torch.log(u))) / tau, -1)
    if hard:
        one_hot = torch.zeros_like(y).scatter_(-1, y.argmax(-1, keepdim=True), 1.0)
        y = one_hot + y - y.detach()
    return y


def score_function_surrogate(log_prob: torch.Tensor, cost: torch.Tensor, baseline: torch.Tensor | float = 0.0) -> torch.Tensor:
    """Surrogate whose gradient is the REINFORCE estimator E[(cost - baseline) grad log p]; add it to the loss."""
    return ((cost - baseline).detach() * log_prob).mean()


# ---- symbolic differentiation ------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class Sym:
    """Expression tree over named variables: ``Sym.var("x")``, constants, + - * / **, sin / cos / exp / log."""
    op: str
    args: tuple = ()

    @staticmethod
    def var(name): return Sym("var", (name,))
    @staticmethod
    def const(v): return Sym("const", (float(v),))
    @staticmethod
    def _w(v): return v if isinstance(v, Sym) else Sym.const(v)
    def __add__(self, o): return Sym("add", (self, Sym._w(o)))
    def __radd__(self, o): return Sym("add", (Sym._w(o), self))
    def __sub__(self, o): return Sym("sub", (self, Sym._w(o)))
    def __rsub__(self, o): return Sym("sub", (Sym._w(o), self))
    def __mul__(self, o): return Sym("mul", (self, Sym._w(o)))
    def __rmul__(self, o): return Sym("mul", (Sym._w(o), self))
    def __truediv__(self, o): return Sym("div", (self, Sym._w(o)))
    def __pow__(self, n): return Sym("pow", (self, Sym._w(n)))
    def __neg__(self): return Sym("mul", (Sym.const(-1.0), self))

    def diff(self, name: str) -> "Sym":
        a = self.args
        if self.op == "const":
            return Sym.const(0)
        if self.op == "var":
            return Sym.const(1.0 if a[0] == name else 0.0)
        if self.op == "add":
            return a[0].diff(name) + a[1].diff(name)
        if self.op == "sub":
            return a[0].diff(name) - a[1].diff(name)
        if self.op == "mul":
            return a[0].diff(name) * a[1] + a[0] * a[1].diff(name)
        if self.op == "div":
            return (a[0].diff(name) * a[1] - a[0] * a[1].diff(name)) / (a[1] * a[1])
        if self.op == "pow":
            return a[1] * a[0] ** (a[1] - 1) * a[0].diff(name)                 # constant exponent
        if self.op == "sin":
            return sym_cos(a[0]) * a[0].diff(name)
        if self.op == "cos":
            return -sym_sin(a[0]) * a[0].diff(name)
        if self.op == "exp":
            return self * a[0].diff(name)
        if self.op == "log":
            return a[0].diff(name) / a[0]
        raise ValueError(self.op)

    def simplify(self) -> "Sym":
        if self.op in ("const", "var"):
            return self
        a = tuple(x.simplify() for x in self.args)
        c = lambda s: s.args[0] if s.op == "const" else None
        if all(x.op == "const" for x in a):
            return Sym.const(Sym(self.op, a).evaluate({}))
        if self.op == "add":
            if c(a[0]) == 0: return a[1]
            if c(a[1]) == 0: return a[0]
        if self.op == "sub" and c(a[1]) == 0:
            return a[0]
        if self.op == "mul":
            if c(a[0]) == 0 or c(a[1]) == 0: return Sym.const(0)
            if c(a[0]) == 1: return a[1]
            if c(a[1]) == 1: return a[0]
        if self.op == "div" and c(a[0]) == 0:
            return Sym.const(0)
        if self.op == "pow":
            if c(a[1]) == 1: return a[0]
            if c(a[1]) == 0: return Sym.const(1)
        return Sym(self.op, a)

    def evaluate(self, env: dict):
        a = self.args
        if self.op == "const": return a[0]
        if self.op == "var": return env[a[0]]
        v = [x.evaluate(env) for x in a]
        t = lambda x: x if isinstance(x, torch.Tensor) else torch.tensor(float(x), dtype=torch.float64)
        return {"add": lambda: v[0] + v[1], "sub": lambda: v[0] - v[1], "mul": lambda: v[0] * v[1], "div": lambda: v[0] / v[1],
                "pow": lambda: v[0] ** v[1], "sin": lambda: torch.sin(t(v[0])), "cos": lambda: torch.cos(t(v[0])),
                "exp": lambda: torch.exp(t(v[0])), "log": lambda: torch.log(t(v[0]))}[self.op]()

    def __str__(self):
        a = self.args
        if self.op == "const": return f"{a[0]:g}"
        if self.op == "var": return a[0]
        sym = {"add": "+", "sub": "-", "mul": "*", "div": "/", "pow": "**"}
        return f"({a[0]} {sym[self.op]} {a[1]})" if self.op in sym else f"{self.op}({a[0]})"


def sym_sin(x): return Sym("sin", (Sym._w(x),))
def sym_cos(x): return Sym("cos", (Sym._w(x),))
def sym_exp(x): return Sym("exp", (Sym._w(x),))
def sym_log(x): return Sym("log", (Sym._w(x),))


# ---- gradient flow analysis and filtering ------------------------------------------------------------------------------
def gradient_flow_report(model: nn.Module, vanish: float = 1e-7, explode: float = 1e3) -> dict:
    """Per-parameter gradient norms after a backward pass, the ratio to the weight norm, and the layers whose gradients
    vanished or exploded."""
    rows = []
    for name, p in model.named_parameters():
        if p.grad is None:
            continue
        g, w = float(p.grad.norm()), float(p.detach().norm())
        rows.append({"name": name, "grad_norm": g, "weight_norm": w, "ratio": g / max(w, 1e-12),
                     "status": "vanishing" if g < vanish else ("exploding" if g > explode or not math.isfinite(g) else "ok")})
    norms = [r["grad_norm"] for r in rows]
    return {"layers": rows, "vanishing": [r["name"] for r in rows if r["status"] == "vanishing"],
            "exploding": [r["name"] for r in rows if r["status"] == "exploding"],
            "max_over_min": (max(norms) / max(min(norms), 1e-30)) if norms else 0.0}


class GradientFilter:
    """Smooths a stream of gradients: exponential moving average, sliding median, or rejection of outliers whose norm is
    more than ``k`` median absolute deviations from the running median (they are replaced by the previous accepted one)."""

    def __init__(self, mode: str = "ema", beta: float = 0.9, window: int = 5, k: float = 5.0):
        self.mode, self.beta, self.window, self.k = mode, beta, window, k
        self.state, self.hist, self.norms, self.rejected = None, deque(maxlen=window), deque(maxlen=50), 0

    def __call__(self, g: torch.Tensor) -> torch.Tensor:
        if self.mode == "ema":
            self.state = g.clone() if self.state is None else self.beta * self.state + (1 - self.beta) * g
            return self.state
        if self.mode == "median":
            self.hist.append(g)
            return torch.stack(list(self.hist)).median(0).values
        if self.mode == "outlier":
            n = float(g.norm())
            if len(self.norms) >= 5:
                med = sorted(self.norms)[len(self.norms) // 2]
                mad = sorted(abs(x - med) for x in self.norms)[len(self.norms) // 2] * 1.4826 + 1e-12
                if abs(n - med) > self.k * mad and self.state is not None:
                    self.rejected += 1
                    return self.state
            self.norms.append(n)
            self.state = g.clone()
            return g
        raise ValueError(self.mode)


def staleness_compensated_gradient(grad: torch.Tensor, w_now: torch.Tensor, w_then: torch.Tensor, lam: float = 0.04) -> torch.Tensor:
    """Delay-compensated asynchronous SGD: a gradient computed at ``w_then`` is corrected towards ``w_now`` with the
    diagonal outer-product approximation of the Hessian, g + lam * g * g * (w_now - w_then)."""
    return grad + lam * grad * grad * (w_now - w_then)


class HypergradientLR:
    """Hypergradient descent (Baydin et al.): the learning rate follows d loss / d lr = - g_t . g_{t-1} for plain SGD."""

    def __init__(self, params, lr: float = 0.01, hyper_lr: float = 1e-4):
        self.params, self.lr, self.hyper_lr, self.prev = list(params), lr, hyper_lr, None

    @torch.no_grad()
    def step(self):
        g = torch.cat([p.grad.reshape(-1) for p in self.params])
        if self.prev is not None:
            self.lr = max(self.lr + self.hyper_lr * float(g @ self.prev), 0.0)
        for p in self.params:
            p -= self.lr * p.grad
        self.prev = g.clone()


class MixedOp(nn.Module):
    """DARTS: softmax(alpha)-weighted sum of candidate operations; ``derive()`` names the strongest one."""

    def __init__(self, ops: dict):
        super().__init__()
        self.names = list(ops)
        self.ops = nn.ModuleList(ops.values())
        self.alpha = nn.Parameter(torch.zeros(len(ops)))

    def forward(self, x):
        w = torch.softmax(self.alpha, 0)
        return sum(wi * op(x) for wi, op in zip(w, self.ops))

    def derive(self) -> str:
        return self.names[int(self.alpha.argmax())]


def autograd_graph_dot(output: torch.Tensor, max_nodes: int = 500) -> str:
    """DOT text of the backward graph reachable from ``output.grad_fn``."""
    lines, seen, stack = ["digraph autograd {", "  rankdir=BT;"], {}, [output.grad_fn]
    while stack and len(seen) < max_nodes:
        fn = stack.pop()
        if fn is None or fn in seen:
            continue
        seen[fn] = len(seen)
        label = type(fn).__name__
        if hasattr(fn, "variable"):
            label += f"\\n{tuple(fn.variable.shape)}"
        lines.append(f'  n{seen[fn]} [label="{label}"];')
        for nxt, _ in fn.next_functions:
            if nxt is not None:
                stack.append(nxt)
    for fn, i in seen.items():
        for nxt, _ in fn.next_functions:
            if nxt in seen:
                lines.append(f"  n{seen[nxt]} -> n{i};")
    return "\n".join(lines + ["}"])


# ---- function transformations in the JAX style (``crates/torsh-autograd/src/jax_transformations.rs``, ``crates/torsh-core/src/jax_transforms.rs``) ----
def grad(fn, argnums=0):
    """``grad(f)(x)`` is the gradient of the scalar ``f`` with respect to the selected positional argument(s); the result is
    itself differentiable, so ``grad(grad(f))`` works."""
    nums = (argnums,) if isinstance(argnums, int) else tuple(argnums)
    def wrapped(*args, **kw):
        args = list(args)
        for n in nums:
            args[n] = args[n] if args[n].requires_grad else args[n].detach().requires_grad_(True)
        out = fn(*args, **kw)
        gs = torch.autograd.grad(out, [args[n] for n in nums], create_graph=True)
        return gs[0] if isinstance(argnums, int) else gs
    return wrapped


def vjp(fn, *primals):
    """``out, pullback = vjp(f, x...)``; ``pullback(cotangent)`` returns one cotangent per primal."""
    xs = [p.detach().requires_grad_(True) for p in primals]
    out = fn(*xs)
    def pullback(ct):
        gs = torch.autograd.grad(out, xs, ct, retain_graph=True, allow_unused=True)
        return tuple(torch.zeros_like(x) if g is None else g for g, x in zip(gs, xs))
    return out.detach(), pullback


def jvp(fn, primals, tangents):
    """Forward-mode: ``(f(x), J v)`` in one pass with dual numbers."""
    import torch.autograd.forward_ad as fwd
    with fwd.dual_level():
        out = fn(*[fwd.make_dual(p, t) for p, t in zip(primals, tangents)])
        o = fwd.unpack_dual(out)
        return o.primal.detach(), (o.tangent if o.tangent is not None else torch.zeros_like(o.primal)).detach()


def jacrev(fn, argnum: int = 0):
    """Jacobian by reverse mode: one batched backward pass per output element (good for few outputs)."""
    def wrapped(*args):
        args = list(args)
        x = args[argnum].detach().requires_grad_(True); args[argnum] = x
        y = fn(*args)
        eye = torch.eye(y.numel(), dtype=y.dtype, device=y.device).reshape(y.numel(), *y.shape)
        j, = torch.autograd.grad(y, x, eye, is_grads_batched=True, create_graph=torch.is_grad_enabled() and y.requires_grad)
        return j.reshape(*y.shape, *x.shape)
    return wrapped


def jacfwd(fn, argnum: int = 0):
    """Jacobian by forward mode: one pass per input element (good for few inputs)."""
    def wrapped(*args):
        x = args[argnum]
        cols = []
        for i in range(x.numel()):
            t = torch.zeros_like(x).reshape(-1); t[i] = 1
            tang = [t.reshape(x.shape) if k == argnum else torch.zeros_like(a) for k, a in enumerate(args)]
            cols.append(jvp(fn, args, tang)[1])
        j = torch.stack(cols, -1)
        return j.reshape(*cols[0].shape, *x.shape)
    return wrapped


def hessian(fn, argnum: int = 0):
    """Forward-over-reverse: the Jacobian (forward mode) of the gradient (reverse mode)."""
    def wrapped(*args):
        x = args[argnum].detach()
        n = x.numel()
        def g(v):
            a = list(args); a[argnum] = v
            return grad(fn, argnum)(*a)
        rows = []
        for i in range(n):
            t = torch.zeros(n, dtype=x.dtype, device=x.device); t[i] = 1
            xv = x.clone().requires_grad_(True)
            gv = g(xv)
            hv, = torch.autograd.grad(gv, xv, t.reshape(x.shape))
            rows.append(hv.reshape(-1))
        return torch.stack(rows).reshape(*x.shape, *x.shape)
    return wrapped


def vmap(fn, in_dims=0, out_dims: int = 0):
    """Maps ``fn`` over one axis of its arguments (``in_dims``: an int for all, or one entry per argument with ``None`` for
    broadcast arguments).  Uses the batching interpreter when the function supports it and an explicit loop otherwise, with
    the same result."""
    def wrapped(*args):
        dims = (in_dims,) * len(args) if isinstance(in_dims, int) or in_dims is None else tuple(in_dims)
        try:
            return torch.vmap(fn, in_dims=dims, out_dims=out_dims)(*args)
        except Exception:                                                           # data-dependent control flow, in-place ops, ...
            n = next(a.shape[d] for a, d in zip(args, dims) if d is not None)
            outs = [fn(*[a.select(d, i) if d is not None else a for a, d in zip(args, dims)]) for i in range(n)]
            if isinstance(outs[0], tuple):
                return tuple(torch.stack([o[k] for o in outs], out_dims) for k in range(len(outs[0])))
            return torch.stack(outs, out_dims)
    return wrapped


def remat(fn):
    """Recomputes ``fn``'s intermediates in the backward pass instead of storing them."""
    from torch.utils.checkpoint import checkpoint
    return lambda *a: checkpoint(fn, *a, use_reentrant=False)


def scan(f, init, xs, reverse: bool = False):
    """``carry, y_t = f(carry, x_t)`` along the first axis; returns the final carry and the stacked ``y``."""
    carry, ys = init, []
    idx = range(len(xs) - 1, -1, -1) if reverse else range(len(xs))
    for i in idx:
        carry, y = f(carry, xs[i]); ys.append(y)
    if reverse:
        ys.reverse()
    return carry, torch.stack(ys) if ys and isinstance(ys[0], torch.Tensor) else ys


def fori_loop(lower: int, upper: int, body, init):
    val = init
    for i in range(lower, upper):
        val = body(i, val)
    return val


def while_loop(cond_fn, body, init, max_iterations: int = 1_000_000):
    val, n = init, 0
    while cond_fn(val):
        val, n = body(val), n + 1
        if n >= max_iterations:
            raise RuntimeError(f"while_loop exceeded {max_iterations} iterations")
    return val


def cond(pred, true_fn, false_fn, *operands):
    """Evaluates one branch for a Python or zero-dimensional predicate; for a batched predicate both branches run and the
    results are selected element-wise (so that the expression stays differentiable and mappable)."""
    if isinstance(pred, torch.Tensor) and pred.dim() > 0:
        a, b = true_fn(*operands), false_fn(*operands)
        return torch.where(pred.reshape(pred.shape + (1,) * (a.dim() - pred.dim())), a, b)
    return true_fn(*operands) if bool(pred) else false_fn(*operands)
