"""metile_b200: the MLX-format affine INT4 projection / fused SwiGLU MLP / add+RMSNorm path of
AndreSlavescu/meTile, written from scratch for NVIDIA B200 (sm_100a).

The operator entry points keep the reference's names and argument order
(`metile_b200.backends`, `metile_b200.kernels`); `metile_b200.compile` is the torch-side
equivalent of `metile.compile`.
"""

from .compile import CompileReport, compile  # noqa: E402,F401  (the function shadows the submodule name)

__all__ = ["compile", "CompileReport"]
