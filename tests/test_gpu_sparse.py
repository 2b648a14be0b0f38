"""GPU parity of the sparse-Jacobian kernels: static gather and index-set algebra (bit-exact ints)."""

import os

import numpy as np
import pytest
import torch

from folx_b200 import masks, sparse
from folx_b200.api import FwdJacobian

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden')
H = np.load(os.path.join(GOLD, 'index_helpers.npz'))


def _names(prefix, suffix):
    return sorted(k[: -len(suffix)] for k in H.files if k.startswith(prefix) and k.endswith(suffix))


@pytest.mark.parametrize('name', _names('mg', '_x'))
def test_gather_matches_reference_static_gather(cuda_device, name):
    x, idx, mx = H[name + '_x'], H[name + '_idx'], int(H[name + '_max'])
    # reference layout is (p, k, r); ours keeps the Jacobian axis first: (k, p, r)
    data = torch.from_numpy(np.ascontiguousarray(np.transpose(x, (1, 0, 2)))).float().to(cuda_device)
    jac = FwdJacobian(data, np.zeros((x.shape[1], x.shape[0], 1), dtype=np.int32))
    got = sparse.materialize_for_idx(jac, np.transpose(idx)[:, :, None], mx)  # (mx, p, r)
    want = np.transpose(H[name + '_out'], (1, 0, 2))
    np.testing.assert_allclose(got.double().cpu().numpy(), want, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize('shape,K,n_in', [((6, 8), 3, 20), ((2, 5, 16), 2, 12), ((4, 3, 2, 32), 4, 9)])
def test_dense_array_of_random_sparse_jacobian(cuda_device, shape, K, n_in):
    rng = np.random.default_rng(1)
    # index map constant along the last axis, unique per position
    idx = np.stack([rng.permutation(n_in)[:K] for _ in range(int(np.prod(shape[:-1])))], axis=-1)
    idx = idx.reshape(K, *shape[:-1], 1).astype(np.int32)
    idx[0].flat[0] = -1
    data = torch.randn((K, *shape), generator=torch.Generator().manual_seed(2))
    jac = FwdJacobian(data.to(cuda_device), idx)
    got = jac.dense_array.cpu().numpy()
    n_rows = int(idx.max()) + 1
    want = np.zeros((n_rows, *shape), dtype=np.float32)
    full = np.broadcast_to(idx, (K, *shape))
    for k in range(K):
        for pos in np.ndindex(*shape):
            t = full[(k, *pos)]
            if t >= 0:
                want[(t, *pos)] += data[(k, *pos)].item()
    assert got.shape == want.shape
    np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-6)


def test_gather_broadcast_input_and_duplicates(cuda_device):
    """Input broadcast along an axis; two stored rows mapping to the same target are summed."""
    data = torch.arange(2 * 1 * 4, dtype=torch.float32).reshape(2, 1, 4).to(cuda_device)
    idx = np.array([[[1], [0], [1]], [[1], [2], [-1]]])  # (2, 3, 1): rows collide at position 0
    jac = FwdJacobian(data, np.zeros((2, 1, 1), dtype=np.int32))
    got = sparse.materialize_for_idx(jac, idx, 3).cpu().numpy()
    d = data.cpu().numpy()
    want = np.zeros((3, 3, 4), dtype=np.float32)
    want[1, 0] = d[0, 0] + d[1, 0]
    want[0, 1] = d[0, 0]; want[2, 1] = d[1, 0]
    want[1, 2] = d[0, 0]
    np.testing.assert_array_equal(got, want)


def test_add_jacobians_rules(cuda_device):
    g = torch.Generator().manual_seed(3)
    a = FwdJacobian(torch.randn(2, 3, 4, generator=g).to(cuda_device), np.array([[[0], [1], [2]], [[3], [4], [5]]]))
    b = FwdJacobian(torch.randn(2, 3, 4, generator=g).to(cuda_device), a.x0_idx.copy())
    s = a + b
    assert s.weak and torch.equal(s.data, a.data + b.data)
    c = FwdJacobian(torch.randn(1, 3, 4, generator=g).to(cuda_device), np.array([[[6], [1], [0]]]))
    s = a + c  # unequal maps: rows are concatenated
    assert s.data.shape[0] == 3 and s.x0_idx.shape == (3, 3, 1)
    np.testing.assert_array_equal(s.x0_idx[2], c.x0_idx[0])
    d = FwdJacobian(torch.randn(9, 3, 4, generator=g).to(cuda_device))
    s = a + d  # dense + sparse: densify and zero-pad
    assert not s.weak and s.data.shape[0] == 9
    torch.testing.assert_close(s.data[:6], a.dense_array + d.data[:6])


@pytest.mark.parametrize('name', _names('su', '_in'))
def test_index_union_kernel_bit_exact(cuda_device, name):
    a = H[name + '_in']
    got = sparse.index_union_device(a, cuda_device)
    want = H[name + '_out']
    assert got.shape == want.shape
    np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize('name', _names('is', '_n'))
def test_index_intersection_kernel_bit_exact(cuda_device, name):
    ms = [H[f'{name}_in{j}'] for j in range(int(H[name + '_n']))]
    got = sparse.index_intersection_device(ms, cuda_device)
    want = H[name + '_out']
    assert got.shape == want.shape
    np.testing.assert_array_equal(got, want)


def test_index_kernels_large_random_against_host(cuda_device):
    rng = np.random.default_rng(5)
    a = rng.integers(-1, 192, size=(64, 64, 24)).astype(np.int32)
    np.testing.assert_array_equal(sparse.index_union_device(a, cuda_device),
                                  masks.per_position_sorted_unique(a))
    parts = [rng.integers(-1, 12, size=(4096, k)).astype(np.int32) for k in (6, 3, 6)]
    np.testing.assert_array_equal(sparse.index_intersection_device(parts, cuda_device),
                                  masks.per_position_intersection(parts))
