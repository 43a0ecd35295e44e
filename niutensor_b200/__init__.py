"""B200-native dense matrix multiplication behind NiuTensor's operator interface.

`capi`  -- ctypes binding of the C ABI (include/ntb_gemm.h), the drop-in boundary.
`ops`   -- host-side mirror of the reference operators of this path (_MatrixMul,
           _MatrixMul2D, _MatrixMulBatched, MatrixMul, MatrixMulBatched/BMMul) over torch
           CUDA tensors; shape rules and error behaviour follow the reference.
`shard` -- column / batch sharding of one product across the ranks of a process group.
"""
from . import capi  # noqa: F401
from .capi import X_TRANS, X_NOTRANS, X_FLOAT, X_FLOAT16  # noqa: F401
