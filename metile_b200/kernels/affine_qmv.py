"""Kernel-level INT4 QMV entry points with the argument order of the reference's eDSL kernels.

Reference: kernels/affine_qmv.py:57 (affine_qmv), :94 (affine_residual_qmv),
:135 (affine_swiglu_qmv), :217 (affine_swiglu_scratch_qmv).  The caller passes the output
tensor; K and N are checked against the tensors; the launch-shape constants BLOCK,
OUTPUTS_PER_SIMDGROUP and HALF_DECODE describe Apple SIMD-group scheduling and are accepted
and ignored.  Rows = X.numel() // K (the reference flattens rows*N outputs the same way).
"""

from __future__ import annotations

from .. import _lib
from ..backends._common import (
    check_affine_triple,
    launch,
    library,
    pointer,
    require_cuda_bf16,
    require_on_device,
)
from ..backends.cuda_quantized import _flags


def _check_io(X, Out, K, N):
    require_cuda_bf16(X, "affine_qmv")
    if X.shape[-1] != K or X.numel() % K:
        raise ValueError("X does not have K columns")
    rows = X.numel() // K
    if Out.dtype != X.dtype or Out.numel() != rows * N or not Out.is_contiguous():
        raise ValueError("Out must be a contiguous [rows, N] tensor of the activation dtype")
    if not X.is_contiguous():
        raise ValueError("X must be contiguous")
    require_on_device(Out, X, "Out", dtype=X.dtype, min_numel=rows * N)
    return rows


def affine_qmv(X, W, Scales, Biases, Out, K, N, GROUP_SIZE=64, BITS=4, BLOCK=32,
               OUTPUTS_PER_SIMDGROUP=1, HALF_DECODE=False):
    del BLOCK, OUTPUTS_PER_SIMDGROUP, HALF_DECODE
    rows = _check_io(X, Out, K, N)
    if check_affine_triple("affine_qmv", X, W, Scales, Biases, GROUP_SIZE, BITS) != N:
        raise ValueError("W does not have N rows")
    code = launch(library().mt_affine_qmv, X.device, pointer(X), pointer(W), pointer(Scales), pointer(Biases), None,
                  pointer(Out), rows, K, N, GROUP_SIZE, BITS, _flags())
    _lib.check(code, "affine_qmv")
    return Out


def affine_residual_qmv(X, W, Scales, Biases, Residual, Out, K, N, GROUP_SIZE=64, BITS=4,
                        BLOCK=32, OUTPUTS_PER_SIMDGROUP=1, HALF_DECODE=False):
    del BLOCK, OUTPUTS_PER_SIMDGROUP, HALF_DECODE
    rows = _check_io(X, Out, K, N)
    if check_affine_triple("affine_residual_qmv", X, W, Scales, Biases, GROUP_SIZE, BITS) != N:
        raise ValueError("W does not have N rows")
    if Residual.numel() != rows * N or Residual.dtype != X.dtype or not Residual.is_contiguous():
        raise ValueError("Residual must be a contiguous [rows, N] tensor of the activation dtype")
    require_on_device(Residual, X, "Residual", dtype=X.dtype, min_numel=rows * N)
    code = launch(library().mt_affine_qmv, X.device, pointer(X), pointer(W), pointer(Scales), pointer(Biases),
                  pointer(Residual), pointer(Out), rows, K, N, GROUP_SIZE, BITS, _flags())
    _lib.check(code, "affine_residual_qmv")
    return Out


def affine_swiglu_qmv(X, GateW, GateScales, GateBiases, UpW, UpScales, UpBiases, Out, K, N,
                      GROUP_SIZE=64, BITS=4, BLOCK=32, OUTPUTS_PER_SIMDGROUP=1, HALF_DECODE=False):
    del BLOCK, OUTPUTS_PER_SIMDGROUP, HALF_DECODE
    rows = _check_io(X, Out, K, N)
    if check_affine_triple("affine_swiglu_qmv", X, GateW, GateScales, GateBiases, GROUP_SIZE,
                           BITS) != N:
        raise ValueError("GateW does not have N rows")
    if check_affine_triple("affine_swiglu_qmv", X, UpW, UpScales, UpBiases, GROUP_SIZE, BITS) != N:
        raise ValueError("UpW does not have N rows")
    code = launch(library().mt_affine_swiglu, X.device, pointer(X), pointer(GateW), pointer(GateScales),
                  pointer(GateBiases), pointer(UpW), pointer(UpScales), pointer(UpBiases), pointer(Out), rows, K, N,
                  GROUP_SIZE, BITS, _flags())
    _lib.check(code, "affine_swiglu_qmv")
    return Out


# The reference's scratch-staged variant returns the same bits as the register-fused one
# (tests/test_mlx_backend.py:1367); here both names run the same kernel.
affine_swiglu_scratch_qmv = affine_swiglu_qmv
