"""Kernel-level RMSNorm with the reference's argument order.

Reference: kernels/rmsnorm.py:5 -- rmsnorm(X, W, Out, N, eps, BLOCK).
"""

from __future__ import annotations

import ctypes

from .. import _lib
from ..backends._common import launch, library, pointer, require_cuda_bf16, require_on_device


def rmsnorm(X, W, Out, N, eps, BLOCK=256):
    del BLOCK
    require_cuda_bf16(X, "rmsnorm")
    if X.shape[-1] != N or W.numel() != N or Out.shape != X.shape or Out.dtype != X.dtype:
        raise ValueError("X, W and Out must agree on N columns")
    for tensor in (X, W, Out):
        if not tensor.is_contiguous():
            raise ValueError("rmsnorm expects contiguous tensors")
    for label, tensor in (("W", W), ("Out", Out)):
        require_on_device(tensor, X, label, dtype=X.dtype)
    code = launch(library().mt_rmsnorm, X.device, pointer(X), pointer(W), pointer(Out), X.numel() // N, N,
                  ctypes.c_float(float(eps)))
    _lib.check(code, "rmsnorm")
    return Out
