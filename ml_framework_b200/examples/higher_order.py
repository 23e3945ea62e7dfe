"""Higher-order-derivative examples, each a function that runs a small problem end to end and returns
the numbers it printed. They mirror the topics of the reference's example set
(src/Examples/HigherOrderDerivatives: MAML, neural ODE, Newton's method, natural gradient,
adversarial robustness, sharpness minimisation) on this framework's autograd facade.

    python -m ml_framework_b200.examples.higher_order [name ...]
"""
from __future__ import annotations

import math
import sys
from typing import Callable, Dict

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..autograd import functional as AF
from ..optim.second_order import NaturalGradient, NewtonCG, hessian_vector_product, power_iteration


def maml(steps: int = 30, inner_lr: float = 0.05, seed: int = 0) -> Dict[str, float]:
    """Model-agnostic meta-learning on sine regression: the outer gradient flows through the inner
    SGD step (a second derivative of the task loss)."""
    g = torch.Generator().manual_seed(seed)
    net = nn.Sequential(nn.Linear(1, 32), nn.Tanh(), nn.Linear(32, 1))
    params = list(net.parameters())
    opt = torch.optim.Adam(params, lr=1e-2)

    def fwd(ws, x):
        return F.linear(torch.tanh(F.linear(x, ws[0], ws[1])), ws[2], ws[3])

    def task():
        amp = 0.5 + 2.0 * torch.rand(1, generator=g)
        ph = math.pi * torch.rand(1, generator=g)
        xs = 6 * torch.rand(20, 1, generator=g) - 3
        return xs[:10], amp * torch.sin(xs[:10] + ph), xs[10:], amp * torch.sin(xs[10:] + ph)

    first = last = 0.0
    for it in range(steps):
        opt.zero_grad()
        meta = 0.0
        for _ in range(4):
            xs, ys, xq, yq = task()
            inner = F.mse_loss(fwd(params, xs), ys)
            grads = torch.autograd.grad(inner, params, create_graph=True)
            adapted = [p - inner_lr * gr for p, gr in zip(params, grads)]
            meta = meta + F.mse_loss(fwd(adapted, xq), yq)
        (meta / 4).backward()
        opt.step()
        if it == 0:
            first = float(meta.detach()) / 4
        last = float(meta.detach()) / 4
    return {"meta_loss_first": first, "meta_loss_last": last}


def neural_ode(steps: int = 60, seed: int = 0) -> Dict[str, float]:
    """Fits dz/dt = f_theta(z) to a damped rotation with a differentiable RK4 integrator and reports
    the Jacobian of the learned vector field at the origin."""
    torch.manual_seed(seed)
    A = torch.tensor([[-0.1, 2.0], [-2.0, -0.1]])
    f = nn.Sequential(nn.Linear(2, 32), nn.Tanh(), nn.Linear(32, 2))

    def rk4(fn, z, h, n):
        out = [z]
        for _ in range(n):
            k1 = fn(z); k2 = fn(z + 0.5 * h * k1); k3 = fn(z + 0.5 * h * k2); k4 = fn(z + h * k3)
            z = z + h / 6 * (k1 + 2 * k2 + 2 * k3 + k4)
            out.append(z)
        return torch.stack(out)

    z0 = torch.tensor([[2.0, 0.0]])
    with torch.no_grad():
        target = rk4(lambda z: z @ A.t(), z0, 0.05, 20)
    opt = torch.optim.Adam(f.parameters(), lr=2e-2)
    first = last = 0.0
    for it in range(steps):
        opt.zero_grad()
        loss = F.mse_loss(rk4(f, z0, 0.05, 20), target)
        loss.backward()
        opt.step()
        first = float(loss.detach()) if it == 0 else first
        last = float(loss.detach())
    J = AF.jacobian(lambda z: f(z), torch.zeros(2))
    return {"loss_first": first, "loss_last": last, "jacobian_trace_at_origin": float(J.diagonal().sum())}


def newton(seed: int = 0) -> Dict[str, float]:
    """Newton-CG on the Rosenbrock function, with the explicit Hessian at the solution."""
    torch.manual_seed(seed)
    x = nn.Parameter(torch.tensor([-1.2, 1.0]))

    def rosen(v=None):
        v = x if v is None else v
        return (1 - v[0]) ** 2 + 100 * (v[1] - v[0] ** 2) ** 2

    opt = NewtonCG([x], lr=1.0, damping=1e-3, cg_iters=20)
    losses = [opt.step(lambda: rosen()) for _ in range(40)]
    H = AF.hessian(rosen, x.detach())
    return {"f_start": losses[0], "f_end": float(rosen().detach()), "hessian_cond": float(torch.linalg.cond(H))}


def natural_gradient(steps: int = 30, seed: int = 0) -> Dict[str, float]:
    """Logistic regression trained with the empirical-Fisher natural gradient."""
    g = torch.Generator().manual_seed(seed)
    X = torch.randn(64, 5, generator=g)
    w_true = torch.randn(5, generator=g)
    y = (X @ w_true > 0).float()
    w = nn.Parameter(torch.zeros(5))
    opt = NaturalGradient([w], lr=0.5, damping=1e-2, cg_iters=20)
    hist = [opt.step(lambda: F.binary_cross_entropy_with_logits(X @ w, y, reduction="none")) for _ in range(steps)]
    acc = float((((X @ w.detach()) > 0).float() == y).float().mean())
    return {"loss_first": hist[0], "loss_last": hist[-1], "accuracy": acc}


def adversarial_robustness(eps: float = 0.1, seed: int = 0) -> Dict[str, float]:
    """FGSM perturbation (gradient w.r.t. the input) and an input-gradient-norm penalty, whose training
    gradient is a second derivative (double back-propagation)."""
    torch.manual_seed(seed)
    X = torch.randn(128, 10)
    y = (X[:, 0] + 0.5 * X[:, 1] > 0).long()
    net = nn.Sequential(nn.Linear(10, 32), nn.Tanh(), nn.Linear(32, 2))
    opt = torch.optim.Adam(net.parameters(), lr=1e-2)
    for _ in range(60):
        opt.zero_grad()
        xi = X.clone().requires_grad_(True)
        loss = F.cross_entropy(net(xi), y)
        gx, = torch.autograd.grad(loss, xi, create_graph=True)
        (loss + 0.5 * gx.pow(2).sum(1).mean() * X.shape[0]).backward()
        opt.step()
    xi = X.clone().requires_grad_(True)
    gx, = torch.autograd.grad(F.cross_entropy(net(xi), y), xi)
    adv = X + eps * gx.sign()
    with torch.no_grad():
        clean = float((net(X).argmax(1) == y).float().mean())
        robust = float((net(adv).argmax(1) == y).float().mean())
    return {"clean_accuracy": clean, "fgsm_accuracy": robust}


def sharpness(seed: int = 0) -> Dict[str, float]:
    """Largest Hessian eigenvalue (power iteration over Hessian-vector products) before and after
    sharpness-aware minimisation steps (gradient taken at the adversarially perturbed weights)."""
    torch.manual_seed(seed)
    X = torch.randn(64, 8)
    y = torch.randn(64, 1)
    net = nn.Sequential(nn.Linear(8, 16), nn.Tanh(), nn.Linear(16, 1))
    params = list(net.parameters())
    n = sum(p.numel() for p in params)
    loss_fn: Callable[[], torch.Tensor] = lambda: F.mse_loss(net(X), y)

    def top_eig():
        lam, _ = power_iteration(lambda v: hessian_vector_product(loss_fn, params, v), n, iters=30)
        return float(lam)

    before = top_eig()
    rho, lr = 0.05, 0.05
    for _ in range(80):
        grads = torch.autograd.grad(loss_fn(), params)
        norm = torch.sqrt(sum(g.pow(2).sum() for g in grads)) + 1e-12
        with torch.no_grad():
            eps = [rho * g / norm for g in grads]
            for p, e in zip(params, eps):
                p.add_(e)
        g2 = torch.autograd.grad(loss_fn(), params)
        with torch.no_grad():
            for p, e, g in zip(params, eps, g2):
                p.sub_(e).sub_(lr * g)
    return {"top_eigenvalue_before": before, "top_eigenvalue_after": top_eig(), "loss": float(loss_fn().detach())}


EXAMPLES = {"maml": maml, "neural_ode": neural_ode, "newton": newton, "natural_gradient": natural_gradient,
            "adversarial_robustness": adversarial_robustness, "sharpness": sharpness}


def main(argv=None):
    names = list(argv if argv is not None else sys.argv[1:]) or list(EXAMPLES)
    for n in names:
        print(n, EXAMPLES[n]())


if __name__ == "__main__":
    main()
