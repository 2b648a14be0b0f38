"""Brute-force Jacobian and Laplacian by automatic differentiation (torch, CPU, fp64).

This is the identity the reference's own tests assert for every rule
(test/laplacian_testcase.py:22-49: ``jacfwd`` for the Jacobian, the trace of the Hessian for the
Laplacian).  The Hessian is taken forward-over-reverse (``torch.func.hessian``).
"""

from __future__ import annotations

from typing import Callable

import torch
from torch.func import hessian, jacfwd, jacrev


def jac_and_laplacian(f: Callable[[torch.Tensor], torch.Tensor], x: torch.Tensor,
                      weights: torch.Tensor | None = None):
    """``(f(x), J, lap)`` with ``J[i] = d f / d x_i`` (shape ``(n, *out)``) and ``lap = tr H``."""
    shape = x.shape
    n = x.numel()

    def flat(z):
        return f(z.reshape(shape))

    x0 = x.reshape(-1)
    y = flat(x0)
    J = jacrev(flat)(x0)  # (*out, n)
    H = hessian(flat)(x0)  # (*out, n, n)
    if weights is not None:
        w = weights.reshape(-1)
        J = J * w
        H = H * w[:, None] * w[None, :]
    lap = torch.diagonal(H, dim1=-2, dim2=-1).sum(-1)
    return y, torch.movedim(J, -1, 0), lap


def propagate(f: Callable[..., torch.Tensor], triplets, n_inputs: int | None = None):
    """Pushes dense triplets through ``f`` by brute force.

    Each triplet ``(x, J, lap)`` is realised as a quadratic map of ``K`` fresh inputs ``t``:
    ``x(t) = x + J . t + 0.5 * lap/K * |t|^2`` has value, Jacobian and Laplacian ``(x, J, lap)`` at
    ``t = 0``; the composition ``f(x(t))`` is then differentiated at 0.
    """
    K = triplets[0][1].shape[0]

    def g(t):
        args = []
        for (x, J, lap) in triplets:
            xt = x + torch.tensordot(t, J, dims=([0], [0])) + 0.5 * lap / K * (t * t).sum()
            args.append(xt)
        return f(*args)

    t0 = torch.zeros(K, dtype=triplets[0][0].dtype)
    return jac_and_laplacian(g, t0)
