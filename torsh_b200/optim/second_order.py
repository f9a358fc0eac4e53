"""Second-order and curvature-aware optimizers of the reference's list (``crates/torsh-optim/src``: Shampoo,
AdaHessian, K-FAC, Newton-CG, YellowFin), written on PyTorch tensors."""
from __future__ import annotations

import torch


def _inv_root(m: torch.Tensor, p: int, eps: float) -> torch.Tensor:
    """``m^(-1/p)`` of a PSD matrix; eigenvalues are floored at ``eps`` times the largest one, so directions the
    statistics have barely seen are not blown up."""
    w, v = torch.linalg.eigh(m)
    floor = max(float(w.max()) * eps, 1e-30)
    return (v * w.clamp(min=floor).pow(-1.0 / p)) @ v.t()


class Shampoo(torch.optim.Optimizer):
    """Per-dimension preconditioners ``L, R`` for matrices (``W -= lr · L^{-1/4} G R^{-1/4}``); vectors fall back to Adagrad."""

    def __init__(self, params, lr=0.03, eps=1e-3, update_freq: int = 10, weight_decay=0.0, max_dim: int = 2048):
        super().__init__(params, dict(lr=lr, eps=eps, update_freq=update_freq, weight_decay=weight_decay, max_dim=max_dim))

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                grad = p.grad.float() + g["weight_decay"] * p.float()
                st = self.state[p]
                mat = grad.reshape(grad.shape[0], -1) if grad.dim() >= 2 else None
                if mat is None or max(mat.shape) > g["max_dim"]:
                    acc = st.setdefault("acc", torch.zeros_like(grad))
                    acc.add_(grad * grad)
                    p.add_((grad / (acc.sqrt() + g["eps"])).to(p.dtype), alpha=-g["lr"])
                    continue
                if not st:
                    st["step"] = 0
                    st["L"] = torch.zeros(mat.shape[0], mat.shape[0], device=p.device)
                    st["R"] = torch.zeros(mat.shape[1], mat.shape[1], device=p.device)
                st["step"] += 1
                st["L"].add_(mat @ mat.t()); st["R"].add_(mat.t() @ mat)
                if st["step"] % g["update_freq"] == 1 or "Li" not in st:
                    st["Li"], st["Ri"] = _inv_root(st["L"], 4, g["eps"]), _inv_root(st["R"], 4, g["eps"])
                p.add_((st["Li"] @ mat @ st["Ri"]).reshape(p.shape).to(p.dtype), alpha=-g["lr"])
        return loss


class AdaHessian(torch.optim.Optimizer):
    """Adam with the squared-gradient moment replaced by a Hutchinson estimate of the Hessian diagonal.
    ``backward(create_graph=True)`` must have produced the gradients."""

    def __init__(self, params, lr=0.1, betas=(0.9, 0.999), eps=1e-4, weight_decay=0.0, hessian_power=1.0):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, hessian_power=hessian_power))

    def _hutchinson(self, params):
        grads = [p.grad for p in params]
        zs = [torch.randint_like(p, 2) * 2 - 1 for p in params]
        hz = torch.autograd.grad(grads, params, grad_outputs=zs, retain_graph=False, allow_unused=True)
        return [(h * z).abs() if h is not None else torch.zeros_like(p) for h, z, p in zip(hz, zs, params)]

    def step(self, closure=None):
        params = [p for g in self.param_groups for p in g["params"] if p.grad is not None and p.grad.requires_grad]
        diag = dict(zip(params, self._hutchinson(params))) if params else {}
        with torch.no_grad():
            for g in self.param_groups:
                b1, b2 = g["betas"]
                for p in g["params"]:
                    if p.grad is None:
                        continue
                    st = self.state[p]
                    if not st:
                        st["step"], st["m"], st["v"] = 0, torch.zeros_like(p), torch.zeros_like(p)
                    st["step"] += 1
                    d = diag.get(p, p.grad.detach().abs())
                    st["m"].mul_(b1).add_(p.grad.detach(), alpha=1 - b1)
                    st["v"].mul_(b2).addcmul_(d, d, value=1 - b2)
                    mh = st["m"] / (1 - b1 ** st["step"]); vh = st["v"] / (1 - b2 ** st["step"])
                    p.mul_(1 - g["lr"] * g["weight_decay"])
                    p.addcdiv_(mh, vh.sqrt().pow(g["hessian_power"]) + g["eps"], value=-g["lr"])
        return None


class KFAC:
    """Kronecker-factored curvature for ``nn.Linear`` layers: ``ΔW = G⁻¹ · dW · A⁻¹`` with running factors
    ``A = E[a aᵀ]`` (inputs) and ``G = E[g gᵀ]`` (output gradients) collected by hooks; other parameters take SGD."""

    def __init__(self, model: torch.nn.Module, lr=0.05, damping=1e-2, ema=0.95, update_freq: int = 5):
        self.model, self.lr, self.damping, self.ema, self.update_freq = model, lr, damping, ema, update_freq
        self.layers = [m for m in model.modules() if isinstance(m, torch.nn.Linear)]
        self.state = {m: {} for m in self.layers}
        self.steps = 0
        for m in self.layers:
            m.register_forward_pre_hook(self._save_input)
            m.register_full_backward_hook(self._save_grad)

    def _save_input(self, m, inp):
        if m.training:
            a = inp[0].detach().reshape(-1, inp[0].shape[-1]).float()
            if m.bias is not None:
                a = torch.cat([a, torch.ones(a.shape[0], 1, device=a.device)], 1)
            self._ema(m, "A", a.t() @ a / a.shape[0])

    def _save_grad(self, m, _gin, gout):
        g = gout[0].detach().reshape(-1, gout[0].shape[-1]).float()
        self._ema(m, "G", g.t() @ g * g.shape[0])

    def _ema(self, m, key, val):
        st = self.state[m]
        st[key] = val if key not in st else self.ema * st[key] + (1 - self.ema) * val

    @torch.no_grad()
    def step(self):
        self.steps += 1
        handled = set()
        for m in self.layers:
            st = self.state[m]
            if m.weight.grad is None or "A" not in st or "G" not in st:
                continue
            if self.steps % self.update_freq == 1 or "Ai" not in st:
                eye = lambda t: self.damping * torch.eye(t.shape[0], device=t.device)
                st["Ai"], st["Gi"] = torch.linalg.inv(st["A"] + eye(st["A"])), torch.linalg.inv(st["G"] + eye(st["G"]))
            dw = m.weight.grad.float()
            if m.bias is not None:
                dw = torch.cat([dw, m.bias.grad.float()[:, None]], 1)
            nat = st["Gi"] @ dw @ st["Ai"]
            m.weight.add_(nat[:, : m.in_features].to(m.weight.dtype), alpha=-self.lr)
            handled.add(m.weight)
            if m.bias is not None:
                m.bias.add_(nat[:, -1].to(m.bias.dtype), alpha=-self.lr); handled.add(m.bias)
        for p in self.model.parameters():
            if p not in handled and p.grad is not None:
                p.add_(p.grad, alpha=-self.lr)

    def zero_grad(self):
        self.model.zero_grad(set_to_none=True)


class NewtonCG:
    """Truncated Newton: solve ``H d = -g`` by conjugate gradient with Hessian-vector products, then ``p += lr · d``."""

    def __init__(self, params, lr=1.0, cg_iters=10, damping=1e-3):
        self.params = [p for p in params if p.requires_grad]
        self.lr, self.cg_iters, self.damping = lr, cg_iters, damping

    def step(self, closure):
        loss = closure()
        grads = torch.autograd.grad(loss, self.params, create_graph=True)
        flat_g = torch.cat([g.reshape(-1) for g in grads])

        def hvp(v):
            hv = torch.autograd.grad(flat_g, self.params, grad_outputs=v, retain_graph=True)
            return torch.cat([h.reshape(-1) for h in hv]) + self.damping * v
        b = -flat_g.detach()
        x, r = torch.zeros_like(b), b.clone()
        p, rs = r.clone(), r @ r
        for _ in range(self.cg_iters):
            hp = hvp(p)
            alpha = rs / (p @ hp).clamp(min=1e-20)
            x, r = x + alpha * p, r - alpha * hp
            rs_new = r @ r
            if rs_new.sqrt() < 1e-10:
                break
            p, rs = r + (rs_new / rs) * p, rs_new
        with torch.no_grad():
            off = 0
            for q in self.params:
                q.add_(x[off:off + q.numel()].view_as(q), alpha=self.lr); off += q.numel()
        return loss.detach()

    def zero_grad(self):
        for p in self.params:
            p.grad = None


class YellowFin(torch.optim.Optimizer):
    """Momentum SGD whose learning rate and momentum are tuned on line from running estimates of the gradient
    variance, the curvature range and the distance to the optimum."""

    def __init__(self, params, lr=1.0, mu=0.0, beta=0.999, window: int = 20):
        super().__init__(params, dict(lr=lr, mu=mu))
        self.beta, self.window, self.h = beta, window, []
        self.g_avg = self.g2_avg = self.dist_avg = self.norm_avg = 0.0
        self.t = 0

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        ps = [p for g in self.param_groups for p in g["params"] if p.grad is not None]
        g2 = float(sum((p.grad.float() ** 2).sum() for p in ps))
        self.t += 1
        b, deb = self.beta, 1 - self.beta ** self.t
        self.h = (self.h + [g2])[-self.window:]
        hmin, hmax = min(self.h), max(self.h)
        self.g2_avg = b * self.g2_avg + (1 - b) * g2
        self.norm_avg = b * self.norm_avg + (1 - b) * g2 ** 0.5
        for p in ps:
            st = self.state[p]
            ga = st.setdefault("g_avg", torch.zeros_like(p, dtype=torch.float32))
            ga.mul_(b).add_(p.grad.float(), alpha=1 - b)
        gbar2 = float(sum((self.state[p]["g_avg"] / deb).pow(2).sum() for p in ps))
        var = max(self.g2_avg / deb - gbar2, 1e-12)
        self.dist_avg = b * self.dist_avg + (1 - b) * (self.norm_avg / deb) / max(self.g2_avg / deb, 1e-12)
        dist = self.dist_avg / deb
        # single-step tuning rule: mu = max(cubic root solution, ((sqrt(hmax/hmin) - 1) / (sqrt(hmax/hmin) + 1))^2)
        pco = dist * dist * hmin * hmin / (2 * var)
        w3 = (-(pco ** 2 + 4.0 / 27.0 * pco ** 3) ** 0.5 - pco) / 2.0
        w = -abs(w3) ** (1.0 / 3.0)
        x = w - pco / 3.0 / w + 1.0
        dr = (hmax / max(hmin, 1e-12)) ** 0.5
        mu = min(max(x * x, ((dr - 1) / (dr + 1)) ** 2), 0.999)
        lr = (1 - mu ** 0.5) ** 2 / max(hmin, 1e-12)
        for g in self.param_groups:
            g["mu"] = b * g["mu"] + (1 - b) * mu
            g["lr"] = b * g["lr"] + (1 - b) * lr if self.t > 1 else min(lr, g["lr"])
            for p in g["params"]:
                if p.grad is None:
                    continue
                buf = self.state[p].setdefault("momentum", torch.zeros_like(p))
                buf.mul_(g["mu"]).add_(p.grad, alpha=-g["lr"])
                p.add_(buf)
        return loss


def _flat(ts):
    return torch.cat([t.reshape(-1) for t in ts])


class TrustRegion:
    """Trust-region Newton method with the Steihaug conjugate-gradient sub-problem
    (``crates/torsh-optim/src/trust_region.rs``): minimise the quadratic model inside a ball of radius ``delta``,
    accept the step when the actual / predicted reduction ratio exceeds ``eta`` and grow or shrink the radius."""

    def __init__(self, params, delta=1.0, max_delta=10.0, eta=0.1, cg_iters=20):
        self.params = [p for p in params if p.requires_grad]
        self.delta, self.max_delta, self.eta, self.cg_iters = delta, max_delta, eta, cg_iters

    def _to_boundary(self, x, d):
        a, b, c = d @ d, 2 * (x @ d), x @ x - self.delta ** 2
        tau = (-b + (b * b - 4 * a * c).clamp(min=0).sqrt()) / (2 * a).clamp(min=1e-30)
        return x + tau * d

    def step(self, closure):
        loss = closure()
        grads = torch.autograd.grad(loss, self.params, create_graph=True)
        g = _flat(grads)

        def hvp(v):
            return _flat(torch.autograd.grad(g, self.params, grad_outputs=v, retain_graph=True))
        gd = g.detach()
        x, r = torch.zeros_like(gd), gd.clone()
        d = -r
        for _ in range(self.cg_iters):
            hd = hvp(d)
            dhd = d @ hd
            if dhd <= 0:                                  # negative curvature: walk to the boundary
                x = self._to_boundary(x, d)
                break
            alpha = (r @ r) / dhd
            xn = x + alpha * d
            if xn.norm() >= self.delta:
                x = self._to_boundary(x, d)
                break
            rn = r + alpha * hd
            x = xn
            if rn.norm() < 1e-10:
                break
            d, r = -rn + ((rn @ rn) / (r @ r)) * d, rn
        predicted = -(gd @ x + 0.5 * (x @ hvp(x)))
        with torch.no_grad():
            off = 0
            for q in self.params:
                q.add_(x[off:off + q.numel()].view_as(q)); off += q.numel()
        new_loss = closure().detach()
        rho = float((loss.detach() - new_loss) / predicted.clamp(min=1e-30))
        if rho < 0.25:
            self.delta *= 0.25
        elif rho > 0.75 and float(x.norm()) >= 0.99 * self.delta:
            self.delta = min(2 * self.delta, self.max_delta)
        if rho <= self.eta:                               # reject: undo the step
            with torch.no_grad():
                off = 0
                for q in self.params:
                    q.sub_(x[off:off + q.numel()].view_as(q)); off += q.numel()
            return loss.detach()
        return new_loss

    def zero_grad(self):
        for p in self.params:
            p.grad = None


class NaturalGradient(torch.optim.Optimizer):
    """Natural-gradient descent with a running diagonal (or, for small tensors, full) empirical Fisher
    (``crates/torsh-optim/src/natural_gradient.rs``): ``F ← β F + (1-β) g gᵀ``, ``p -= lr (F + λ I)⁻¹ g``."""

    def __init__(self, params, lr=0.1, beta=0.95, damping=1e-3, full_below: int = 0):
        super().__init__(params, dict(lr=lr, beta=beta, damping=damping, full_below=full_below))

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for grp in self.param_groups:
            for p in grp["params"]:
                if p.grad is None:
                    continue
                g = p.grad.float().reshape(-1)
                st = self.state[p]
                st["t"] = st.get("t", 0) + 1
                deb = 1 - grp["beta"] ** st["t"]
                if g.numel() <= grp["full_below"]:
                    f = st.setdefault("fisher", torch.zeros(g.numel(), g.numel(), device=g.device))
                    f.mul_(grp["beta"]).add_(torch.outer(g, g), alpha=1 - grp["beta"])
                    nat = torch.linalg.solve(f / deb + grp["damping"] * torch.eye(g.numel(), device=g.device), g)
                else:
                    f = st.setdefault("fisher_diag", torch.zeros_like(g))
                    f.mul_(grp["beta"]).addcmul_(g, g, value=1 - grp["beta"])
                    nat = g / (f / deb + grp["damping"])
                p.add_(nat.view_as(p).to(p.dtype), alpha=-grp["lr"])
        return loss
