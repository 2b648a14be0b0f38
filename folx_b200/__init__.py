"""folx_b200 -- forward-Laplacian propagation on NVIDIA B200 (sm_100a).

A drop-in for the forward-Laplacian hot path of microsoft/folx: the same public names
(reference: folx/__init__.py:1-24) over hand-written CUDA kernels behind a C ABI.
"""

from .api import (  # noqa: F401
    JAC_DIM,
    FunctionFlags,
    FwdJacobian,
    FwdLaplArgs,
    FwdLaplArray,
)

__version__ = '0.1.0'
