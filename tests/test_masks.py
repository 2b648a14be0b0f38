"""Index-map algebra (host NumPy) against the golden fixtures.

``index_helpers.npz`` holds outputs of the reference's own NumPy helpers on seeded inputs and
``find_out_idx_cases.json`` the literal known-answer cases of the reference's
test/test_find_out_idx.py; both are produced by tests/golden/make_golden.py.  Bit-exact.
"""

import json
import os

import numpy as np
import pytest

from folx_b200 import masks
from folx_b200.api import FunctionFlags

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden')
H = np.load(os.path.join(GOLD, 'index_helpers.npz'))
CASES = json.load(open(os.path.join(GOLD, 'find_out_idx_cases.json')))['cases']


def _keys(prefix, suffix):
    return sorted(k[: -len(suffix)] for k in H.files if k.startswith(prefix) and k.endswith(suffix))


@pytest.mark.parametrize('name', _keys('su', '_in'))
def test_sorted_unique_matches_reference(name):
    got = masks.per_position_sorted_unique(H[name + '_in'])
    want = H[name + '_out']
    assert got.shape == want.shape and got.dtype == want.dtype
    np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize('name', _keys('is', '_n'))
def test_intersection_matches_reference(name):
    ms = [H[f'{name}_in{j}'] for j in range(int(H[name + '_n']))]
    got = masks.per_position_intersection(ms)
    want = H[name + '_out']
    assert got.shape == want.shape
    np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize('name', _keys('dup', '_in'))
def test_duplicate_detection(name):
    assert masks.has_duplicate_x0_idx(H[name + '_in']) == bool(H[name + '_out'])
    assert masks.has_duplicate_x0_idx(None) is False


@pytest.mark.parametrize('name', _keys('cr', '_in'))
def test_compaction(name):
    got, axes = masks.compact_repeated_dims_except(H[name + '_in'], 0)
    np.testing.assert_array_equal(got, H[name + '_out'])
    assert tuple(axes) == tuple(H[name + '_axes'])


@pytest.mark.parametrize('name', _keys('mg', '_x'))
def test_gather_table_reproduces_the_static_gather(name):
    x, idx, mx = H[name + '_x'], H[name + '_idx'], int(H[name + '_max'])
    take = masks.gather_table(idx, mx)  # (p, max_idx, n_slots)
    p = x.shape[0]
    got = np.zeros((p, mx, x.shape[2]))
    for s in range(take.shape[2]):
        t = take[:, :, s]
        rows = np.take_along_axis(x, np.maximum(t, 0)[:, :, None], axis=1)
        got += np.where((t >= 0)[:, :, None], rows, 0.0)
    np.testing.assert_allclose(got, H[name + '_out'], atol=1e-12)
    # every valid source row is used exactly once
    used = np.sort(np.concatenate([take[q][take[q] >= 0] for q in range(p)]))
    want_used = np.sort(np.concatenate([np.nonzero(idx[q] >= 0)[0] for q in range(p)]))
    np.testing.assert_array_equal(used, want_used)


def _run_case(case):
    if 'arange_mask' in case:
        ms = [np.arange(np.prod(case['arange_mask']), dtype=np.int32).reshape(case['arange_mask'])]
    else:
        ms = [np.asarray(m, dtype=np.int32) for m in case['masks']]
    shapes = [tuple(s) for s in case['x_shapes']] if 'x_shapes' in case else [m.shape[1:] for m in ms]
    return masks.find_out_idx(ms, shapes, [tuple(a) for a in case['in_axes']],
                              FunctionFlags[case['flags']], case['threshold'])


@pytest.mark.parametrize('case', CASES, ids=[c['src'] for c in CASES])
def test_find_out_idx_known_answers(case):
    idx, dense = _run_case(case)
    assert dense is case['dense']
    if 'expected' in case:
        want = np.asarray(case['expected'], dtype=np.int64)
        assert idx.shape == want.shape, (idx.shape, want.shape)
        np.testing.assert_array_equal(idx, want)
    if 'expected_shape' in case:
        assert list(idx.shape) == case['expected_shape']
    if 'expected_shape_tail' in case:
        assert list(idx.shape[1:]) == case['expected_shape_tail']
    if 'expected_rows' in case:
        assert idx.shape[0] == case['expected_rows']
    if 'expected_col0' in case:
        np.testing.assert_array_equal(idx[:, 0], case['expected_col0'])
    for pos, want in case.get('expected_sets', {}).items():
        i, j = (int(v) for v in pos.split(','))
        assert sorted(int(v) for v in idx[:, i, j] if v >= 0) == want


def test_find_out_idx_dense_only():
    idx, dense = masks.find_out_idx([None], [(4,)], [()], FunctionFlags.GENERAL, 10, dense_rows=[3])
    assert idx is None and dense is True


def test_get_index_mask_first_match_and_padding():
    mask = np.array([[0, 5], [3, -1], [0, 7]])
    outputs = np.array([[0, 5], [3, 7], [-1, -1]])
    got = masks.get_index_mask(mask, outputs)
    # row 1, position 1 is -1 and matches the first -1 padding slot, as in the reference
    np.testing.assert_array_equal(got, [[0, 0], [1, 2], [0, 1]])
    assert masks.get_index_mask(mask, np.zeros((0, 2), dtype=int)).tolist() == [[-1, -1]] * 3


def test_reduction_frame_first_dense_layer_of_the_readme_mlp():
    """x:(100,4) with identity map, contracting axis 1 -> K=4, out_mask[c, i] = 4 i + c."""
    x0 = np.arange(400).reshape(1, 100, 4)
    out_mask, (targets,) = masks.reduction_frame([x0], (1,))
    assert out_mask.shape == (4, 100)
    np.testing.assert_array_equal(out_mask, (4 * np.arange(100)[None, :] + np.arange(4)[:, None]))
    # stored row 0 at (i, c) lands in output row c
    np.testing.assert_array_equal(targets[0], np.broadcast_to(np.arange(4)[None, :], (100, 4)))


def test_sum_outdeps_pairwise_distances():
    """sum over the coordinate axis of (r_i - r_j)^2: 6 rows off the diagonal, 3 on it."""
    N = 3
    i, j, c = np.meshgrid(np.arange(N), np.arange(N), np.arange(3), indexing='ij')
    m = np.stack([3 * i + c, 3 * j + c])  # (2, N, N, 3)
    idx_out, targets = masks.sum_outdeps(m, (2,))
    assert idx_out.shape == (6, N, N)
    for a in range(N):
        for b in range(N):
            want = sorted({3 * a + k for k in range(3)} | {3 * b + k for k in range(3)})
            assert [v for v in idx_out[:, a, b] if v >= 0] == want
    assert (idx_out[3:, 0, 0] == -1).all()
    assert targets.shape == (2, N, N, 3)


def test_union_rows_order_is_lexicographic():
    m1 = np.array([[3, 4, 5]])
    m2 = np.array([[0, 1, 2]])
    res, inv = masks.union_rows([m1, m2])
    np.testing.assert_array_equal(res, [[0, 1, 2], [3, 4, 5]])
    assert inv.tolist() == [1, 0]


# ---- factor tables of the sparse log-determinant rule (folx/slogdet.py:93-293) ---------------------
def _slogdet_mask(mode, n):
    if mode == 'entries':
        return np.stack([np.roll(np.arange(n), s) for s in range(n)])[None].astype(np.int64)
    mask = np.zeros((3, n, n), dtype=np.int64)
    for k in range(3):
        mask[k] = (3 * np.arange(n) + k)[:, None]
    if mode == 'two_rows':
        mask = np.concatenate([mask, np.roll(mask, 1, axis=1)], axis=0)
    if mode == 'columns':
        mask = np.swapaxes(mask, -1, -2).copy()
    if mode == 'shared':
        mask = np.broadcast_to(np.arange(3 * n).reshape(3 * n, 1, 1), (3 * n, n, n)).copy()
    return mask


@pytest.mark.parametrize('mode,fast,shape', [
    ('rows', True, (18, 1, 6)), ('two_rows', True, (18, 2, 6)), ('columns', True, (18, 1, 6)),
    ('entries', True, (6, 6, 1)), ('shared', False, None)])
def test_sparse_slogdet_plan_follows_the_reference_cases(mode, fast, shape):
    """Which masks take the factorised rule and with which table shape (the cases of the
    reference's test/test_layers.py:340-420: rows, two rows, columns, single entries, no structure)."""
    n = 6
    mask = _slogdet_mask(mode, n)
    plan = masks.plan_sparse_slogdet(mask, (n, n), int(mask.max()) + 1)
    assert (plan is not None) == fast
    if fast:
        take, cols, rows, coords, transposed = plan
        assert take.shape == shape and cols.shape == shape and rows.shape == shape[:2]
        assert transposed == (mode == 'columns')
        np.testing.assert_array_equal(coords, np.arange(int(mask.max()) + 1))
    # the same map stored once for a batch of walkers (size-1 batch axes) plans identically,
    # whatever the batch extent of the values
    batched = masks.plan_sparse_slogdet(mask.reshape(mask.shape[0], 1, 1, n, n), (4096, 16, n, n),
                                        int(mask.max()) + 1)
    assert (batched is not None) == fast


@pytest.mark.parametrize('mode', ['rows', 'two_rows', 'columns', 'entries'])
def test_sparse_slogdet_tables_reproduce_the_rule(mode):
    """The contraction the kernel runs on the tables, W_c[s, t] = sum_l dA[take] A^-1[cols, rows]
    (A^-1 read transposed for column factors), written in NumPy: J_c = tr W_c and
    lap = tr(A^-1 lapA) - sum_c tr(W_c W_c) must equal the dense rule on the densified Jacobian."""
    rng = np.random.default_rng(5)
    n = 5
    mask = _slogdet_mask(mode, n)
    k = mask.shape[0]
    n_in = int(mask.max()) + 1
    A = rng.normal(size=(n, n)) + 2 * np.eye(n)
    J = rng.normal(size=(k, n, n))
    lapA = rng.normal(size=(n, n))
    take, cols, rows, coords, transposed = masks.plan_sparse_slogdet(mask, (n, n), n_in) or \
        (*masks.slogdet_factor_tables(mask, False)[1:], False)
    C = np.linalg.inv(A)
    flat = np.concatenate([J.reshape(-1), [0.0]])
    vals = flat[np.where(take >= 0, take, J.size)]                       # (coords, rank, width)
    Cg = C[rows[:, None, None, :], cols[..., None]] if transposed else C[cols[..., None], rows[:, None, None, :]]
    W = np.einsum('csl,cslt->cst', vals, Cg)
    jac = np.zeros(n_in)
    jac[coords] = np.einsum('css->c', W)
    lap = np.einsum('ji,ij->', C, lapA) - np.einsum('cst,cts->', W, W)
    dense = np.zeros((n_in, n, n))
    for s in range(k):
        for i in range(n):
            for j in range(n):
                dense[mask[s, i, j], i, j] += J[s, i, j]
    M = C @ dense
    np.testing.assert_allclose(jac, np.einsum('kii->k', M), rtol=1e-10, atol=1e-12)
    np.testing.assert_allclose(lap, np.einsum('ji,ij->', C, lapA) - np.einsum('kij,kji->', M, M), rtol=1e-10)
