"""Residual add + RMSNorm and RMSNorm on CUDA, behind the reference's operator names.

Reference: metile/backends/mlx.py:786-830 (mlx_add_rms_norm) and :748-783 (mlx_rms_norm).
The reference runs a timing tournament between block sizes and native MLX; here there is one
hand-written kernel per op, so `autotune` is accepted and ignored.
"""

from __future__ import annotations

import ctypes

import torch

from .. import _lib
from ._common import launch, library, pointer, require_cuda_bf16, require_on_device, rows_of


def mlx_rms_norm(values, weight, eps, *, autotune=True):
    """RMSNorm over the last axis: bf16(x * rsqrt(mean(x^2) + eps) * w)."""
    del autotune
    if values.ndim < 1 or weight.ndim != 1 or values.shape[-1] != weight.shape[0]:
        raise ValueError("meTile RMSNorm requires a matching one-dimensional weight")
    if values.dtype != weight.dtype:
        raise TypeError("meTile RMSNorm requires matching input and weight dtypes")
    require_cuda_bf16(values, "meTile RMSNorm")
    require_on_device(weight, values, "RMSNorm weight", contiguous=False)
    x = values.contiguous()
    w = weight.contiguous()
    out = torch.empty_like(x)
    if x.numel() == 0:
        return out
    code = launch(library().mt_rmsnorm, x.device, pointer(x), pointer(w), pointer(out), rows_of(x), x.shape[-1],
                  ctypes.c_float(float(eps)))
    _lib.check(code, "mlx_rms_norm")
    return out


def mlx_add_rms_norm(values, residual, weight, eps, *, autotune=True):
    """Fused residual add + RMSNorm; returns (summed, normalized)."""
    del autotune
    if values.shape != residual.shape or values.dtype != residual.dtype:
        raise ValueError("meTile fused add/RMSNorm requires matching residual inputs")
    if values.ndim < 1 or weight.ndim != 1 or values.shape[-1] != weight.shape[0]:
        raise ValueError("meTile fused add/RMSNorm requires a matching RMSNorm weight")
    if values.dtype != weight.dtype:
        raise TypeError("meTile fused add/RMSNorm requires matching input and weight dtypes")
    require_cuda_bf16(values, "meTile fused add/RMSNorm")
    require_on_device(residual, values, "residual", contiguous=False)
    require_on_device(weight, values, "RMSNorm weight", contiguous=False)
    x = values.contiguous()
    r = residual.contiguous()
    w = weight.contiguous()
    summed = torch.empty_like(x)
    normalized = torch.empty_like(x)
    if x.numel() == 0:
        return summed, normalized
    code = launch(library().mt_add_rmsnorm, x.device, pointer(x), pointer(r), pointer(w), pointer(summed),
                  pointer(normalized), rows_of(x), x.shape[-1], ctypes.c_float(float(eps)))
    _lib.check(code, "mlx_add_rms_norm")
    return summed, normalized
