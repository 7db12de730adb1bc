"""Multi-row affine INT4 matmul behind the reference's `MLXAffineWeight` / `mlx_affine_matmul`.

Reference: metile/backends/mlx_affine.py:66-114 (MLXAffineWeight) and :359-406
(mlx_affine_matmul).  The reference keeps a K-major repacked copy of the weights for Apple's
matrix unit and accepts float16 only; the CUDA kernels read the MLX layout directly, so the
weight object holds just the native arrays and the activations are bfloat16.
"""

from __future__ import annotations

from dataclasses import dataclass

from .cuda_quantized import mlx_affine_qmv


@dataclass(frozen=True)
class MLXAffineWeight:
    """One MLX affine uint4 weight: packed words, scales, biases and its logical (K, N) shape."""

    native_weight: object
    native_scales: object
    native_biases: object
    shape: tuple
    group_size: int = 64
    bits: int = 4

    @classmethod
    def from_mlx(cls, weight, scales, biases, *, group_size=64, bits=4):
        if group_size != 64 or bits != 4:
            raise ValueError(
                f"MLX affine weights require group size 64 and 4 bits, got {group_size} and {bits}."
            )
        if biases is None:
            raise ValueError("native affine QMV requires affine biases")
        if weight.ndim != 2 or scales.ndim != 2 or biases.shape != scales.shape:
            raise ValueError("expected packed weight and matching two-dimensional parameters")
        input_features = weight.shape[1] * 32 // bits
        return cls(weight, scales, biases, (input_features, weight.shape[0]), group_size, bits)

    # The reference exposes the repacked arrays under these names; here they alias the native ones.
    @property
    def packed(self):
        return self.native_weight

    @property
    def scales(self):
        return self.native_scales

    @property
    def biases(self):
        return self.native_biases


def mlx_affine_matmul(values, weight, *, autotune=True):
    """values [..., K] @ dequant(weight)^T -> [..., N]; ragged row counts are handled in-kernel."""
    del autotune
    if not isinstance(weight, MLXAffineWeight):
        raise TypeError("mlx_affine_matmul expects an MLXAffineWeight")
    if values.shape[-1] != weight.shape[0]:
        raise ValueError("activation width does not match the affine weight")
    return mlx_affine_qmv(values, weight.native_weight, weight.native_scales, weight.native_biases,
                          group_size=weight.group_size, bits=weight.bits)
