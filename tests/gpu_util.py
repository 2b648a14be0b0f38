"""Helpers shared by the GPU parity tests: seeded triplets on both sides of the comparison."""

import numpy as np
import torch

from folx_b200 import kernels
from folx_b200.api import FwdJacobian, FwdLaplArray

RTOL = 1e-4  # BASELINE.json: x / J / laplacian within rtol 1e-4 in fp32


def seeded_triplet(K, shape, seed=0, positive=False, scale=1.0):
    """(x, J, lap) in fp64 on the CPU from a fixed seed."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, dtype=torch.float64, generator=g) * scale
    if positive:
        x = x.abs() + 0.5
    J = torch.randn((K, *shape), dtype=torch.float64, generator=g)
    lap = torch.randn(shape, dtype=torch.float64, generator=g)
    # round to fp32 so both sides see identical inputs
    return tuple(t.float().double() for t in (x, J, lap))


def to_device(t, device, x0_idx=None, stacked=True) -> FwdLaplArray:
    x, J, lap = t
    K = J.shape[0]
    if stacked:
        out = kernels.alloc_triplet(K, x.shape, device, x0_idx)
        out.x.copy_(x.float())
        out.jacobian.data.copy_(J.float())
        out.laplacian.copy_(lap.float())
        return out
    return FwdLaplArray(x.float().to(device), FwdJacobian(J.float().to(device), x0_idx),
                        lap.float().to(device))


def to_host(a: FwdLaplArray):
    return (a.x.double().cpu(), a.jacobian.data.double().cpu(), a.laplacian.double().cpu())


def assert_close(got, want, rtol=RTOL, atol_scale=1e-5):
    """rtol 1e-4 with an absolute floor scaled to the magnitude of each tensor."""
    for g, w, name in zip(got, want, ('x', 'jacobian', 'laplacian')):
        atol = atol_scale * max(float(w.abs().max()), 1e-30) if w.numel() else 0.0
        torch.testing.assert_close(g, w, rtol=rtol, atol=atol, msg=lambda m: f'{name}: {m}')
