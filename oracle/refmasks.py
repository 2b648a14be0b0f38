"""Executes the reference's pure-NumPy index-map helpers from a checkout of the reference.

TEST INFRASTRUCTURE ONLY, and only for generating fixtures: ``tests/golden/make_golden.py`` uses it
on a machine that has the reference checkout; the tests themselves read the committed fixtures.
Nothing is copied: the named ``FunctionDef`` nodes are parsed out of the reference's files and
executed in a namespace where ``jnp`` is NumPy (the helpers only touch static integer masks) and
``jax.tree_util`` is a two-function shim.
"""

from __future__ import annotations

import ast
import os
import types
from typing import Sequence

import numpy as np

WANTED = {
    'folx/hessian.py': ['_has_duplicate_x0_idx', '_vmap_axes_to_original', '_align_mask_for_broadcast',
                        '_per_position_sorted_unique', '_per_position_intersection'],
    'folx/utils.py': ['bound_axis', 'materialize_by_gather', 'compact_repeated_dims_except',
                      'broadcast_except'],
    'folx/slogdet.py': ['_slots', '_factor_tables'],
}


class _TreeShim:
    @staticmethod
    def tree_leaves(x):
        return list(x) if isinstance(x, (list, tuple)) else [x]

    @staticmethod
    def tree_map(fn, x):
        return type(x)(fn(v) for v in x) if isinstance(x, (list, tuple)) else fn(x)


def load(reference_root: str) -> types.SimpleNamespace:
    ns: dict = {'np': np, 'jnp': np, 'jtu': _TreeShim, 'JAC_DIM': 0, 'Sequence': Sequence,
                '_MAX_MASK_ENTRIES': 2**24}
    for rel, names in WANTED.items():
        path = os.path.join(reference_root, rel)
        tree = ast.parse(open(path).read(), filename=path)
        picked = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in names]
        missing = set(names) - {n.name for n in picked}
        if missing:
            raise RuntimeError(f'{rel}: functions not found: {sorted(missing)}')
        mod = ast.Module(body=picked, type_ignores=[])
        exec(compile(mod, path, 'exec'), ns)
    return types.SimpleNamespace(**{n: ns[n] for names in WANTED.values() for n in names})
