"""CUDA backends: torch-tensor operator entry points with the reference's names and signatures."""

from .cuda import (  # noqa: F401
    mlx_add_rms_norm,
    mlx_attention_decode,
    mlx_rms_norm,
    rope_kv_append,
    supports_attention_decode,
)
from .cuda_affine import MLXAffineWeight, mlx_affine_matmul  # noqa: F401
from .cuda_dense import (  # noqa: F401
    mlx_dense_residual_qmv,
    mlx_dense_swiglu,
)
from .cuda_quantized import (  # noqa: F401
    batch_invariant,
    force_kernel,
    mlx_affine_mlp_executor,
    mlx_affine_mlp_host_executor,
    mlx_affine_qmv,
    mlx_affine_residual_qmv,
    mlx_affine_residual_qmv_dispatches,
    mlx_affine_swiglu,
    mlx_affine_swiglu_dispatches,
    mlx_affine_swiglu_executor,
    mlx_affine_swiglu_qmv,
    repack_mlx_affine_weight,
)
