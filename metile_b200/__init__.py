"""metile_b200: the MLX-format affine INT4 projection / fused SwiGLU MLP / add+RMSNorm path of
AndreSlavescu/meTile, written from scratch for NVIDIA B200 (sm_100a).

The operator entry points keep the reference's names and argument order
(`metile_b200.backends`, `metile_b200.kernels`); `metile_b200.compile` is the torch-side
equivalent of `metile.compile`.
"""

__all__ = ["compile", "CompileReport"]


def __getattr__(name):
    if name in ("compile", "CompileReport"):
        import importlib

        module = importlib.import_module(".compile", __name__)
        return getattr(module, name)
    raise AttributeError(name)
