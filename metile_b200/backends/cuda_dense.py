"""Dense bf16 small-batch projections whose rows are bit-identical to running each row alone.

Reference: metile/backends/mlx_dense_residual.py and metile/backends/mlx_dense_swiglu.py (the
rows < 32 SIMD-group kernels lowered by metile/compiler/dense.py:193-381).  Weights are plain
row-major bf16 [N, K]; K must be a multiple of 128.
"""

from __future__ import annotations

import torch

from .. import _lib
from ._common import contiguous_2d, launch, library, pointer, require_cuda_bf16, require_on_device


def _check_dense(name, values, weight):
    require_cuda_bf16(values, name)
    if weight.ndim != 2 or weight.shape[1] != values.shape[-1]:
        raise ValueError(f"{name} expects a [N, K] weight matching the activation width")
    if weight.dtype != values.dtype:
        raise TypeError(f"{name} requires matching activation and weight dtypes")
    if values.shape[-1] % 128:
        raise ValueError(f"{name} requires the input width to be a multiple of 128")
    if not weight.is_contiguous() or weight.device != values.device:
        raise ValueError(f"{name} expects a contiguous weight on the activation's device")


def mlx_dense_residual_qmv(values, weight, residual=None):
    """bf16(bf16(values @ weight^T) + residual); residual may be None."""
    name = "dense residual projection"
    _check_dense(name, values, weight)
    expected = (*values.shape[:-1], weight.shape[0])
    if residual is not None and (tuple(residual.shape) != expected or residual.dtype != values.dtype):
        raise ValueError("residual must match the projection output shape and dtype")
    require_on_device(residual, values, "residual", contiguous=False)
    x = contiguous_2d(values)
    res = None if residual is None else contiguous_2d(residual)
    out = torch.empty((x.shape[0], weight.shape[0]), dtype=values.dtype, device=values.device)
    code = launch(library().mt_dense_rows, values.device, pointer(x), pointer(weight), pointer(res), pointer(out),
                  x.shape[0], x.shape[1], weight.shape[0])
    _lib.check(code, name)
    return out.reshape(expected)


def mlx_dense_swiglu(values, gate_weight, up_weight):
    """Typed SwiGLU of two dense projections (each rounded to bf16 before the activation)."""
    name = "dense SwiGLU"
    _check_dense(name, values, gate_weight)
    _check_dense(name, values, up_weight)
    if gate_weight.shape != up_weight.shape:
        raise ValueError("dense SwiGLU requires matching gate/up weights")
    x = contiguous_2d(values)
    out = torch.empty((x.shape[0], gate_weight.shape[0]), dtype=values.dtype, device=values.device)
    code = launch(library().mt_dense_swiglu, values.device, pointer(x), pointer(gate_weight), pointer(up_weight),
                  pointer(out), x.shape[0], x.shape[1], gate_weight.shape[0])
    _lib.check(code, name)
    return out.reshape(*values.shape[:-1], gate_weight.shape[0])
