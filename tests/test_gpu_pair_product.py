"""GPU parity of the one-pass product of two triplets (fl_dot_general_pair) against the oracle's
restatement of the reference rule (dot_general of two non-constant operands,
folx/wrapped_functions.py:205-309, Hessian term folx/hessian.py:177-188), plus properties at a
walker-scale batch."""

import pytest
import torch

from folx_b200 import kernels
from folx_b200 import rules as dev_rules
from oracle import rules

from gpu_util import assert_close, seeded_triplet, to_device, to_host

pytestmark = pytest.mark.gpu


@pytest.fixture(params=[0, 1], ids=['auto', 'fp32-pipe'], autouse=True)
def pair_mode(request):
    """Every case runs with the kernel chosen by shape (tensor cores for square 16- and 32-wide
    products) and with the fp32-pipe kernel forced."""
    from folx_b200 import lib
    lib.load().fl_dot_general_pair_set_mode(request.param)
    yield request.param
    lib.load().fl_dot_general_pair_set_mode(0)


@pytest.mark.parametrize('m,c,n', [(1, 1, 1), (4, 4, 4), (16, 16, 16), (3, 5, 7), (17, 9, 6), (8, 32, 12),
                                   (32, 32, 32), (64, 64, 64), (5, 130, 3), (64, 3, 64),
                                   (32, 16, 16), (48, 16, 16), (64, 16, 16), (16, 32, 32), (48, 32, 32),
                                   (64, 32, 32), (16, 64, 16), (16, 16, 64), (32, 64, 32), (64, 32, 64),
                                   (48, 64, 64), (16, 32, 16), (32, 16, 32)])
@pytest.mark.parametrize('K,batch', [(0, (3,)), (5, (7,)), (19, (2, 3))])
def test_pair_product_matches_oracle(cuda_device, m, c, n, K, batch):
    a = seeded_triplet(K, (*batch, m, c), seed=m + 3 * c + K)
    b = seeded_triplet(K, (*batch, c, n), seed=n + 5 * c + K + 1)
    assert kernels.pair_product_fits(m, c, n)
    got = kernels.dot_general_pair(to_device(a, cuda_device), to_device(b, cuda_device))
    assert_close(to_host(got), rules.dot_general_pair(a, b), rtol=1e-4, atol_scale=2e-5)


@pytest.mark.parametrize('m,c,n', [(8, 12, 8), (16, 16, 16), (32, 32, 32)])
@pytest.mark.parametrize('shared', ['a', 'b'])
def test_pair_product_with_one_matrix_shared_by_the_batch(cuda_device, shared, m, c, n):
    K = 6
    a = seeded_triplet(K, ((1, 1) if shared == 'a' else (3, 5)) + (m, c), seed=1)
    b = seeded_triplet(K, ((1, 1) if shared == 'b' else (3, 5)) + (c, n), seed=2)
    got = kernels.dot_general_pair(to_device(a, cuda_device), to_device(b, cuda_device))
    assert_close(to_host(got), rules.dot_general_pair(a, b), rtol=1e-4, atol_scale=2e-5)


def test_pair_product_on_views_and_unequal_row_counts(cuda_device):
    """The rule pads the shorter Jacobian with zero rows and copies strided views."""
    K, m, c, n = 7, 6, 10, 4
    a = seeded_triplet(K, (5, c, m), seed=3)
    b = seeded_triplet(K - 3, (5, c, n), seed=4)
    at = (a[0].transpose(-1, -2), a[1].transpose(-1, -2), a[2].transpose(-1, -2))
    da = to_device(a, cuda_device)
    da = dev_rules.permute(da, (0, 2, 1))
    got = dev_rules.dot_general_pair(da, to_device(b, cuda_device))
    bp = (b[0], torch.cat([b[1], torch.zeros(3, *b[1].shape[1:], dtype=b[1].dtype)]), b[2])
    assert_close(to_host(got), rules.dot_general_pair(at, bp), rtol=1e-4, atol_scale=2e-5)


def test_oversized_pair_is_refused(cuda_device):
    from folx_b200 import lib
    assert not kernels.pair_product_fits(128, 16, 128)
    a = to_device(seeded_triplet(1, (1, 128, 16), seed=5), cuda_device)
    b = to_device(seeded_triplet(1, (1, 16, 128), seed=6), cuda_device)
    with pytest.raises(RuntimeError, match='do not fit'):
        kernels.dot_general_pair(a, b)
    # the rule takes the product-and-sum route instead
    got = dev_rules.dot_general_pair(a, b)
    assert tuple(got.x.shape) == (1, 128, 128)


def test_pair_product_properties_at_walker_scale(cuda_device):
    """4096 walkers x 16 x 16 x 16, K = 48: linear in either operand's derivatives, and a constant
    right operand reproduces the one-operand product."""
    g = torch.Generator(device=cuda_device).manual_seed(9)
    K, B, d = 48, 4096, 16
    rnd = lambda *s: torch.randn(*s, generator=g, device=cuda_device)

    def trip(shape):
        t = kernels.alloc_triplet(K, shape, cuda_device, None)
        t.x.copy_(rnd(*shape)); t.jacobian.data.copy_(rnd(K, *shape)); t.laplacian.copy_(rnd(*shape))
        return t

    a, b = trip((B, d, d)), trip((B, d, d))
    y = kernels.dot_general_pair(a, b)
    torch.testing.assert_close(y.x, a.x @ b.x, rtol=1e-4, atol=1e-4)
    want_j = a.jacobian.data @ b.x + a.x @ b.jacobian.data
    torch.testing.assert_close(y.jacobian.data, want_j, rtol=1e-4, atol=2e-4)
    want_l = a.laplacian @ b.x + a.x @ b.laplacian + 2 * (a.jacobian.data @ b.jacobian.data).sum(0)
    torch.testing.assert_close(y.laplacian, want_l, rtol=1e-4, atol=2e-3)
    # a constant b (zero derivatives): only the terms of the one-operand rule remain
    b.jacobian.data.zero_(); b.laplacian.zero_()
    y0 = kernels.dot_general_pair(a, b)
    torch.testing.assert_close(y0.jacobian.data, a.jacobian.data @ b.x, rtol=1e-4, atol=2e-4)
    torch.testing.assert_close(y0.laplacian, a.laplacian @ b.x, rtol=1e-4, atol=2e-4)
