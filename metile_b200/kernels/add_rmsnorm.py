"""Kernel-level residual add + RMSNorm with the reference's argument order.

Reference: kernels/add_rmsnorm.py:5 -- add_rmsnorm(X, Residual, W, Sum, Out, N, eps, BLOCK).
N is the row width; BLOCK is an Apple threadgroup size, accepted and ignored.
"""

from __future__ import annotations

import ctypes

from .. import _lib
from ..backends._common import launch, library, pointer, require_cuda_bf16, require_on_device


def add_rmsnorm(X, Residual, W, Sum, Out, N, eps, BLOCK=256):
    del BLOCK
    require_cuda_bf16(X, "add_rmsnorm")
    if X.shape[-1] != N or W.numel() != N:
        raise ValueError("X and W must have N columns")
    for tensor in (Residual, Sum, Out):
        if tensor.shape != X.shape or tensor.dtype != X.dtype:
            raise ValueError("Residual, Sum and Out must match X")
    for tensor in (X, Residual, W, Sum, Out):
        if not tensor.is_contiguous():
            raise ValueError("add_rmsnorm expects contiguous tensors")
    for label, tensor in (("Residual", Residual), ("W", W), ("Sum", Sum), ("Out", Out)):
        require_on_device(tensor, X, label, dtype=X.dtype)
    code = launch(library().mt_add_rmsnorm, X.device, pointer(X), pointer(Residual), pointer(W), pointer(Sum),
                  pointer(Out), X.numel() // N, N, ctypes.c_float(float(eps)))
    _lib.check(code, "add_rmsnorm")
    return Sum, Out
