"""The workspace-free local-energy entry point against the regular one.

``fl_local_energy_static`` serves callers that cannot supply scratch memory or allocate (a custom
call inside a compiler-planned step, a host whose framework owns all device memory): its partial
sums live in a fixed array inside the library.  Because that array is shared by every call and
keeps its old contents, the check runs the entry point twice in a row -- with different sizes, so
the second call finds leftovers of the first -- and compares both results with
``fl_local_energy``.  This file sorts last on purpose: a run that stops at the first failure has
then already executed every other test.
"""

import ctypes

import pytest
import torch

from folx_b200 import kernels, lib

pytestmark = pytest.mark.gpu


def _ptr(t):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _static(lap, jac, pot):
    B, K = lap.numel(), jac.shape[0]
    energy = torch.empty(B, dtype=torch.float32, device=lap.device)
    sums = torch.empty(3, dtype=torch.float64, device=lap.device)
    stream = ctypes.c_void_p(torch.cuda.current_stream(lap.device).cuda_stream)
    lib.call('fl_local_energy_static', _ptr(lap), _ptr(jac), max(B, 1), _ptr(pot), B, K,
             _ptr(energy), _ptr(sums), stream)
    return energy, sums


def test_static_scratch_variant_matches_on_two_consecutive_calls(cuda_device):
    g = torch.Generator().manual_seed(11)
    for B, K in ((5000, 48), (777, 96)):  # the second, smaller call sees the first call's leftovers
        lap = torch.randn(B, generator=g).to(cuda_device)
        jac = torch.randn(K, B, generator=g).to(cuda_device)
        pot = torch.randn(B, generator=g).to(cuda_device)
        want_e, want_s = kernels.local_energy(lap, jac, pot)
        got_e, got_s = _static(lap, jac, pot)
        torch.testing.assert_close(got_e, want_e, rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(got_s, want_s, rtol=1e-12, atol=1e-9)


def test_static_scratch_variant_rejects_oversized_batches(cuda_device):
    handle = lib.load()
    too_many = 1048576 + 1
    rc = handle.fl_local_energy_static(None, None, too_many, None, too_many, 0, None,
                                       ctypes.c_void_p(8), None)
    assert rc == lib.FL_EBADSHAPE
    assert b'exceed the built-in scratch' in handle.fl_last_error()
