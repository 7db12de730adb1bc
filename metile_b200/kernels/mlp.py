"""Kernel-level MLP entry points.

Reference: kernels/mlp.py:34 (matmul_silu) and :7 (matmul_gelu) -- dense C = act(A @ B) with
A [M, K], B [K, N], C [M, N]; tile sizes are tuning constants there and are ignored here.
Served for bfloat16 at M <= 128; larger M is refused, not rerouted.

`affine_swiglu_mlp` is the fused quantized MLP (gate|up SwiGLU -> down, + residual) with the
argument order of metile/backends/mlx_quantized.py:1770 (mlx_affine_mlp_executor), output and
hidden workspace passed by the caller.
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


def _matmul_act(name, A, B, C, M, N, K, flags):
    require_cuda_bf16(A, name)
    if tuple(A.shape) != (M, K) or tuple(B.shape) != (K, N) or tuple(C.shape) != (M, N):
        raise ValueError(f"{name} expects A [M,K], B [K,N], C [M,N]")
    if B.dtype != A.dtype or C.dtype != A.dtype:
        raise TypeError(f"{name} requires matching dtypes")
    if M > 128:
        raise ValueError(f"{name} serves M <= 128 rows")
    for tensor in (A, B, C):
        if not tensor.is_contiguous():
            raise ValueError(f"{name} expects contiguous tensors")
    require_on_device(B, A, "B", dtype=A.dtype, min_numel=K * N)
    require_on_device(C, A, "C", dtype=A.dtype, min_numel=M * N)
    code = launch(library().mt_dense_act, A.device, pointer(A), pointer(B), pointer(C), M, N, K, flags)
    _lib.check(code, name)
    return C


def matmul_silu(A, B, C, M, N, K, BLOCK_M=None, BLOCK_N=None, BLOCK_K=None):
    """C = SiLU(A @ B)."""
    del BLOCK_M, BLOCK_N, BLOCK_K
    return _matmul_act("matmul_silu", A, B, C, M, N, K, 0)


def matmul_gelu(A, B, C, M, N, K, BLOCK_M=None, BLOCK_N=None, BLOCK_K=None):
    """C = A@B / (1 + exp(-1.702 * A@B))."""
    del BLOCK_M, BLOCK_N, BLOCK_K
    return _matmul_act("matmul_gelu", A, B, C, M, N, K, _lib.FLAG_GELU)


def affine_swiglu_mlp(X, GateW, GateScales, GateBiases, UpW, UpScales, UpBiases, DownW, DownScales,
                      DownBiases, Residual, Hidden, Out, GROUP_SIZE=64, BITS=4):
    """Out = down(swiglu(X)) + Residual; Hidden [rows, I] bf16 is caller-owned scratch."""
    name = "affine_swiglu_mlp"
    require_cuda_bf16(X, name)
    hidden_features = X.shape[-1]
    rows = X.numel() // hidden_features
    intermediate = check_affine_triple(name, X, GateW, GateScales, GateBiases, GROUP_SIZE, BITS)
    check_affine_triple(name, X, UpW, UpScales, UpBiases, GROUP_SIZE, BITS)
    if check_affine_triple(name, Hidden, DownW, DownScales, DownBiases, GROUP_SIZE,
                           BITS) != hidden_features:
        raise ValueError("down projection must map back to the input width")
    if Hidden.numel() < rows * intermediate or Out.numel() != rows * hidden_features:
        raise ValueError("Hidden or Out has the wrong size")
    for tensor in (X, Hidden, Out) + (() if Residual is None else (Residual,)):
        if not tensor.is_contiguous():
            raise ValueError(f"{name} expects contiguous tensors")
    require_on_device(Hidden, X, "Hidden", dtype=X.dtype, min_numel=rows * intermediate)
    require_on_device(Out, X, "Out", dtype=X.dtype, min_numel=rows * hidden_features)
    require_on_device(Residual, X, "Residual", dtype=X.dtype, min_numel=rows * hidden_features)
    if Residual is not None and Residual.numel() != rows * hidden_features:
        raise ValueError("Residual must be a [rows, hidden] tensor")
    code = launch(
        library().mt_affine_mlp, X.device, pointer(X), pointer(GateW), pointer(GateScales), pointer(GateBiases),
        pointer(UpW), pointer(UpScales), pointer(UpBiases), pointer(DownW), pointer(DownScales),
        pointer(DownBiases), pointer(Residual), pointer(Hidden), Hidden.numel() * 2, pointer(Out),
        rows, hidden_features, intermediate, GROUP_SIZE, BITS, _flags())
    _lib.check(code, name)
    return Out
