"""Second-order optimisers and their linear-algebra helpers.

Reference: src/MLFramework/Optimizers/SecondOrder/{LBFGS,Newton,NaturalGradient,HessianAwareAdam}Optimizer.cs,
ConjugateGradientSolver.cs, PowerIteration.cs. All of them need curvature-vector products; those come from
double backward (Hessian-vector product) without forming the Hessian.
"""
from __future__ import annotations

from collections import deque
from typing import Callable, Deque, Iterable, List, Sequence, Tuple

import torch


def _flat(ts: Sequence[torch.Tensor]) -> torch.Tensor:
    return torch.cat([t.reshape(-1) for t in ts])


def _unflat(v: torch.Tensor, like: Sequence[torch.Tensor]) -> List[torch.Tensor]:
    out, o = [], 0
    for t in like:
        out.append(v[o:o + t.numel()].view_as(t))
        o += t.numel()
    return out


def hessian_vector_product(loss_fn: Callable[[], torch.Tensor], params: Sequence[torch.Tensor], v: torch.Tensor) -> torch.Tensor:
    loss = loss_fn()
    g = _flat(torch.autograd.grad(loss, params, create_graph=True))
    hv = torch.autograd.grad(g @ v, params, allow_unused=True)
    return _flat([h if h is not None else torch.zeros_like(p) for h, p in zip(hv, params)]).detach()


def conjugate_gradient(matvec: Callable[[torch.Tensor], torch.Tensor], b: torch.Tensor, max_iter: int = 50, tol: float = 1e-6,
                       damping: float = 0.0) -> Tuple[torch.Tensor, int, float]:
    """Solves (A + damping I) x = b for symmetric positive-definite A given only products with A."""
    x = torch.zeros_like(b)
    r = b.clone()
    p = r.clone()
    rs = r @ r
    it = 0
    for it in range(1, max_iter + 1):
        Ap = matvec(p) + damping * p
        denom = p @ Ap
        if denom <= 0:                              # negative curvature: stop with what we have
            if it == 1:
                x = b.clone()
            break
        alpha = rs / denom
        x = x + alpha * p
        r = r - alpha * Ap
        rs_new = r @ r
        if rs_new.sqrt() < tol:
            rs = rs_new
            break
        p = r + (rs_new / rs) * p
        rs = rs_new
    return x, it, float(rs.sqrt())


def power_iteration(matvec: Callable[[torch.Tensor], torch.Tensor], dim: int, iters: int = 50, tol: float = 1e-5,
                    device=None, dtype=torch.float32, seed: int = 0) -> Tuple[float, torch.Tensor]:
    """Largest-magnitude eigenvalue / vector of a symmetric operator."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    v = torch.randn(dim, generator=g, dtype=dtype).to(device or "cpu")
    v = v / v.norm()
    lam = 0.0
    for _ in range(iters):
        w = matvec(v)
        new = float(v @ w)
        n = w.norm()
        if n == 0:
            return 0.0, v
        v = w / n
        if abs(new - lam) <= tol * max(1.0, abs(new)):
            lam = new
            break
        lam = new
    return lam, v


class _Base:
    def __init__(self, params: Iterable[torch.nn.Parameter]):
        self.params = [p for p in params]

    def zero_grad(self):
        for p in self.params:
            p.grad = None

    def _set(self, flat: torch.Tensor):
        with torch.no_grad():
            for p, v in zip(self.params, _unflat(flat, self.params)):
                p.copy_(v)

    def _get(self) -> torch.Tensor:
        return _flat([p.detach() for p in self.params]).clone()


class LBFGS(_Base):
    """Two-loop recursion with a backtracking Armijo line search. ``step(closure)``: closure returns the loss
    (with grad enabled; it is re-evaluated during the line search)."""

    def __init__(self, params, lr: float = 1.0, history: int = 10, max_ls: int = 20, c1: float = 1e-4):
        super().__init__(params)
        self.lr, self.max_ls, self.c1 = lr, max_ls, c1
        self.s: Deque[torch.Tensor] = deque(maxlen=history)
        self.y: Deque[torch.Tensor] = deque(maxlen=history)
        self._prev_g = self._prev_x = None

    def _grad(self, closure):
        self.zero_grad()
        loss = closure()
        g = _flat(torch.autograd.grad(loss, self.params))
        return float(loss.detach()), g

    def step(self, closure: Callable[[], torch.Tensor]) -> float:
        f, g = self._grad(closure)
        x = self._get()
        if self._prev_g is not None:
            s, y = x - self._prev_x, g - self._prev_g
            if float(s @ y) > 1e-10:
                self.s.append(s)
                self.y.append(y)
        q = g.clone()
        alphas = []
        for s, y in zip(reversed(self.s), reversed(self.y)):
            a = (s @ q) / (y @ s)
            alphas.append(a)
            q -= a * y
        if self.s:
            q *= (self.s[-1] @ self.y[-1]) / (self.y[-1] @ self.y[-1])
        for (s, y), a in zip(zip(self.s, self.y), reversed(alphas)):
            b = (y @ q) / (y @ s)
            q += (a - b) * s
        d = -q
        gd = float(g @ d)
        if gd >= 0:
            d, gd = -g, -float(g @ g)
        t = self.lr
        for _ in range(self.max_ls):
            self._set(x + t * d)
            with torch.no_grad():
                fn = float(closure())
            if fn <= f + self.c1 * t * gd:
                break
            t *= 0.5
        self._prev_x, self._prev_g = x, g
        return f


class NewtonCG(_Base):
    """Newton step from conjugate gradient on Hessian-vector products, with Levenberg damping."""

    def __init__(self, params, lr: float = 1.0, damping: float = 1e-3, cg_iters: int = 50, cg_tol: float = 1e-6):
        super().__init__(params)
        self.lr, self.damping, self.cg_iters, self.cg_tol = lr, damping, cg_iters, cg_tol

    def step(self, closure):
        loss = closure()
        g = _flat(torch.autograd.grad(loss, self.params)).detach()
        d, _, _ = conjugate_gradient(lambda v: hessian_vector_product(closure, self.params, v), g, self.cg_iters, self.cg_tol, self.damping)
        self._set(self._get() - self.lr * d)
        return float(loss.detach())


class NaturalGradient(_Base):
    """Preconditions the gradient with the empirical Fisher F = E[g_i g_i^T] (+ damping) through CG;
    ``per_sample_losses`` returns a vector of losses, one per sample."""

    def __init__(self, params, lr: float = 0.1, damping: float = 1e-2, cg_iters: int = 20):
        super().__init__(params)
        self.lr, self.damping, self.cg_iters = lr, damping, cg_iters

    def step(self, per_sample_losses: Callable[[], torch.Tensor]):
        losses = per_sample_losses()
        G = torch.stack([_flat(torch.autograd.grad(l, self.params, retain_graph=True)) for l in losses])   # [n, P]
        g = G.mean(0)
        d, _, _ = conjugate_gradient(lambda v: G.t() @ (G @ v) / G.shape[0], g, self.cg_iters, 1e-8, self.damping)
        self._set(self._get() - self.lr * d)
        return float(losses.mean())


class HessianAwareAdam(_Base):
    """Adam whose second moment tracks Hutchinson estimates of the Hessian diagonal (z * Hz, z = +-1)
    instead of squared gradients."""

    def __init__(self, params, lr: float = 1e-2, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0, hessian_every: int = 1, seed: int = 0):
        super().__init__(params)
        self.lr, self.betas, self.eps, self.wd, self.k = lr, betas, eps, weight_decay, hessian_every
        n = sum(p.numel() for p in self.params)
        dev = self.params[0].device
        self.m, self.v, self.t = torch.zeros(n, device=dev), torch.zeros(n, device=dev), 0
        self.gen = torch.Generator(device="cpu").manual_seed(seed)
        self._diag = torch.zeros(n, device=dev)

    def step(self, closure):
        loss = closure()
        g = _flat(torch.autograd.grad(loss, self.params)).detach()
        if self.t % self.k == 0:
            z = (torch.randint(0, 2, (g.numel(),), generator=self.gen).float() * 2 - 1).to(g.device)
            self._diag = (z * hessian_vector_product(closure, self.params, z)).abs()
        self.t += 1
        b1, b2 = self.betas
        self.m.mul_(b1).add_(g, alpha=1 - b1)
        self.v.mul_(b2).addcmul_(self._diag, self._diag, value=1 - b2)
        mh, vh = self.m / (1 - b1 ** self.t), self.v / (1 - b2 ** self.t)
        x = self._get()
        x = x * (1 - self.lr * self.wd) - self.lr * mh / (vh.sqrt() + self.eps)
        self._set(x)
        return float(loss.detach())
