"""Data model of the forward Laplacian: the (x, Jacobian, Laplacian) triplet.

Mirrors the reference's containers (folx/api.py:16-464): same field names, same meaning, the
Jacobian axis first (``JAC_DIM = 0``), sparse Jacobians as ``k`` rows plus a static NumPy index
map ``x0_idx`` (``-1`` marks an unused row).  Arrays are ``torch`` CUDA tensors; index maps are
NumPy ``int32`` arrays that live on the host and are broadcast-compatible with ``data``.
"""

from __future__ import annotations

from enum import IntFlag
from typing import Any, Callable, NamedTuple, Protocol

import numpy as np
import torch

JAC_DIM = 0  # reference: folx/api.py:16

Array = torch.Tensor


class FwdJacobian(NamedTuple):
    """Jacobian of a tensor w.r.t. the function's inputs (reference: folx/api.py:19-263).

    ``data`` has shape ``(k, *shape)``.  Dense: ``x0_idx is None`` and row ``i`` is the derivative
    w.r.t. input ``i``.  Sparse: ``x0_idx[(k, ...)]`` names the input each row belongs to.
    """

    data: Array
    x0_idx: np.ndarray | None = None

    @property
    def weak(self) -> bool:
        return self.x0_idx is not None

    @property
    def unique_idx(self) -> np.ndarray:
        if self.x0_idx is not None:
            return np.unique(self.x0_idx)
        return np.arange(self.data.shape[JAC_DIM])

    @property
    def data_shape(self) -> tuple[int, ...]:
        return tuple(self.data.shape[1:])

    @property
    def max_n(self) -> int:
        if self.x0_idx is not None:
            return int(np.max(self.x0_idx))
        return self.data.shape[JAC_DIM]

    @property
    def mask(self) -> np.ndarray:
        """Index map; for a dense Jacobian it is ``arange(k)`` broadcast over the positions."""
        if self.x0_idx is not None:
            return self.x0_idx
        k = self.data.shape[JAC_DIM]
        ext = (slice(None),) + (None,) * (self.data.ndim - 1)
        return np.broadcast_to(np.arange(k, dtype=np.int32)[ext], tuple(self.data.shape))

    @property
    def ndim(self) -> int:
        return self.data.ndim

    @classmethod
    def from_dense(cls, array: Array) -> 'FwdJacobian':
        return cls(array, None)

    def materialize_for_idx(self, idx: np.ndarray, max_idx: int | None = None) -> Array:
        """Rows gathered/summed into the frame ``idx`` (reference: folx/api.py:58-118)."""
        from . import sparse

        return sparse.materialize_for_idx(self, idx, max_idx)

    def get_index_mask(self, outputs: np.ndarray) -> np.ndarray:
        """For every stored row the position of its input in ``outputs`` or -1 (folx/api.py:120-159)."""
        from . import masks

        return masks.get_index_mask(self.mask, outputs)

    def construct_jac_for(self, idx) -> Array:
        """Jacobian rows for the inputs listed in ``idx`` (reference: folx/api.py:165-180)."""
        if idx is None:
            return self.dense_array
        idx = np.asarray(idx)
        if len(idx) == 0:
            return torch.zeros((1, *self.data_shape), dtype=self.data.dtype, device=self.data.device)
        if self.x0_idx is None:
            return self.data[torch.as_tensor(idx.reshape(-1), device=self.data.device)]
        return self.materialize_for_idx(self.get_index_mask(idx), len(idx))

    @property
    def dense_array(self) -> Array:
        """Dense Jacobian with ``max_n + 1`` rows (reference: folx/api.py:182-190)."""
        if self.x0_idx is None:
            return self.data
        # the frame 0 .. max_n holds input v in slot v, so the slot of every stored row is its
        # own map entry (what get_index_mask would find by comparison)
        return self.materialize_for_idx(np.where(self.x0_idx >= 0, self.x0_idx, -1).astype(np.int64),
                                        self.max_n + 1)

    @property
    def as_dense(self) -> 'FwdJacobian':
        return FwdJacobian.from_dense(self.dense_array)

    @property
    def dense_or_sparse(self) -> Array:
        return self.data

    @property
    def sparse(self) -> Array:
        assert self.weak
        return self.data

    def __add__(self, other):  # type: ignore[override]
        """Sum of two Jacobians (reference: folx/api.py:230-249)."""
        assert isinstance(other, FwdJacobian)
        from . import sparse

        return sparse.add_jacobians(self, other)

    def astype(self, dtype) -> 'FwdJacobian':
        return FwdJacobian(self.data.to(dtype), self.x0_idx)


class FwdLaplArray(NamedTuple):
    """Triplet of a tensor, its Jacobian and its Laplacian (reference: folx/api.py:266-333)."""

    x: Array
    jacobian: FwdJacobian
    laplacian: Array

    @property
    def shape(self):
        return tuple(self.x.shape)

    @property
    def ndim(self):
        return self.x.ndim

    @property
    def size(self):
        return self.x.numel()

    @property
    def dense_jacobian(self):
        return self.jacobian.dense_array

    @property
    def is_jacobian_weak(self):
        return self.jacobian.weak

    @property
    def sparse_jacobian(self):
        return self.jacobian.sparse

    @property
    def jacobian_mask(self):
        return self.jacobian.mask

    @property
    def dense(self):
        return FwdLaplArray(self.x, self.jacobian.as_dense, self.laplacian)

    @property
    def dtype(self):
        return self.x.dtype

    def astype(self, dtype):
        if dtype.is_floating_point:
            return FwdLaplArray(self.x.to(dtype), self.jacobian.astype(dtype), self.laplacian.to(dtype))
        # integer / boolean targets drop the derivatives (reference: folx/api.py:317-318)
        return self.x.to(dtype)


def IS_LPL_ARR(x) -> bool:
    return isinstance(x, FwdLaplArray)


class FwdLaplArgs(NamedTuple):
    """A tuple of triplets with per-field accessors (reference: folx/api.py:348-409)."""

    arrays: tuple[FwdLaplArray, ...]

    @property
    def x(self):
        return tuple(a.x for a in self.arrays)

    @property
    def jacobian(self):
        return tuple(a.jacobian for a in self.arrays)

    @property
    def dense_jacobian(self):
        return tuple(a.dense_jacobian for a in self.arrays)

    @property
    def sparse_jacobian(self):
        return tuple(a.sparse_jacobian for a in self.arrays)

    @property
    def jacobian_mask(self):
        return tuple(a.jacobian_mask for a in self.arrays)

    @property
    def all_jacobian_weak(self) -> bool:
        return all(a.is_jacobian_weak for a in self.arrays)

    @property
    def any_jacobian_weak(self) -> bool:
        return any(a.is_jacobian_weak for a in self.arrays)

    @property
    def dense(self):
        return FwdLaplArgs(tuple(a.dense for a in self.arrays))

    @property
    def laplacian(self):
        return tuple(a.laplacian for a in self.arrays)

    def __len__(self) -> int:
        return len(self.arrays)


class ForwardLaplacian(Protocol):
    """Signature of a registered rule (reference: folx/api.py:444-450)."""

    def __call__(self, args: tuple, kwargs: dict[str, Any], sparsity_threshold: int) -> Any: ...


class CustomTraceJacHessianJac(Protocol):
    """Signature of a custom tr(J^T H J) hook (reference: folx/api.py:434-441)."""

    def __call__(self, args: FwdLaplArgs, extra_args: tuple, merge: Callable, materialize_idx) -> Any: ...


class FunctionFlags(IntFlag):
    """Structure hints of a wrapped function (reference: folx/api.py:453-464)."""

    GENERAL = 0
    LINEAR_IN_FIRST = 1 << 0
    LINEAR_IN_ONE = 1 << 1 | LINEAR_IN_FIRST
    LINEAR = 1 << 2 | LINEAR_IN_ONE
    REDUCTION = 1 << 3
    MULTIPLICATION = 1 << 4 | LINEAR_IN_ONE
    DOT_PRODUCT = 1 << 5 | REDUCTION | MULTIPLICATION
    INDEXING = 1 << 6 | LINEAR
    SCATTER = 1 << 7
    SPARSE_JHJ = 1 << 8
    SUMMATION = 1 << 9 | LINEAR | REDUCTION
