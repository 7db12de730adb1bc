"""CPU tests of the drop-in boundary: the shared library loads, exports every symbol the header
declares, and rejects bad arguments before touching a GPU."""

import ctypes
import os
import re

import pytest

from metile_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "metile_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mt_[a-z_0-9]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_lib.LIBRARY_PATH)
    names = declared_symbols()
    assert "mt_affine_mlp" in names and "mt_add_rmsnorm" in names and len(names) >= 13
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/metile_b200.h but not exported"
    assert set(_lib.SIGNATURES) <= set(names)


def test_status_strings_and_version():
    lib = _lib.load()
    assert lib.mt_version() >= 100
    assert _lib.status_string(0) == "ok"
    for code in range(-8, 0):
        assert _lib.status_string(code) != "unknown status"


def test_arguments_are_validated_before_any_gpu_work():
    lib = _lib.load()
    one = ctypes.c_void_p(16)
    # 8-bit format and group 32 are refused (MT_ERR_FORMAT) whatever the pointers are.
    assert lib.mt_affine_qmv(one, one, one, one, None, one, 1, 64, 64, 32, 4, 0, None) == -3
    assert lib.mt_affine_qmv(one, one, one, one, None, one, 1, 64, 64, 64, 8, 0, None) == -3
    # K not a multiple of 64.
    assert lib.mt_affine_qmv(one, one, one, one, None, one, 1, 96, 64, 64, 4, 0, None) == -1
    # Null pointers.
    assert lib.mt_affine_qmv(None, one, one, one, None, one, 1, 64, 64, 64, 4, 0, None) == -6
    # Misaligned activation pointer.
    assert lib.mt_affine_qmv(ctypes.c_void_p(18), one, one, one, None, one, 1, 64, 64, 64, 4, 0, None) == -2
    # Workspace too small for the MLP.
    assert lib.mt_affine_mlp(*([one] * 10), None, one, 16, one, 4, 64, 64, 64, 4, 0, None) == -7
    assert lib.mt_affine_mlp_workspace_bytes(4, 2048, 8192) == 4 * 8192 * 2
    with pytest.raises(ValueError):
        _lib.check(-3, "probe")
    with pytest.raises(RuntimeError):
        _lib.check(-4, "probe")


def test_operator_signatures_match_the_reference():
    import inspect

    from metile_b200 import backends
    from metile_b200.kernels import add_rmsnorm, affine_qmv, mlp, rmsnorm

    def names(function):
        return list(inspect.signature(function).parameters)

    assert names(backends.mlx_affine_qmv) == ["values", "weight", "scales", "biases", "group_size", "bits",
                                              "block", "outputs_per_simdgroup", "decode_dtype"]
    assert names(backends.mlx_affine_residual_qmv) == ["values", "weight", "scales", "biases", "residual",
                                                       "group_size", "bits", "autotune"]
    assert names(backends.mlx_affine_swiglu)[:7] == ["values", "gate_weight", "gate_scales", "gate_biases",
                                                     "up_weight", "up_scales", "up_biases"]
    assert names(backends.mlx_affine_mlp_executor)[:11] == [
        "sample_values", "gate_weight", "gate_scales", "gate_biases", "up_weight", "up_scales", "up_biases",
        "down_weight", "down_scales", "down_biases", "sample_residual"]
    assert names(backends.mlx_add_rms_norm) == ["values", "residual", "weight", "eps", "autotune"]
    assert names(backends.mlx_rms_norm) == ["values", "weight", "eps", "autotune"]
    assert names(affine_qmv.affine_qmv)[:7] == ["X", "W", "Scales", "Biases", "Out", "K", "N"]
    assert names(affine_qmv.affine_swiglu_qmv)[:10] == ["X", "GateW", "GateScales", "GateBiases", "UpW",
                                                         "UpScales", "UpBiases", "Out", "K", "N"]
    assert names(add_rmsnorm.add_rmsnorm) == ["X", "Residual", "W", "Sum", "Out", "N", "eps", "BLOCK"]
    assert names(rmsnorm.rmsnorm) == ["X", "W", "Out", "N", "eps", "BLOCK"]
    assert names(mlp.matmul_silu)[:6] == ["A", "B", "C", "M", "N", "K"]


def test_operators_refuse_cpu_tensors_and_bad_formats():
    import torch

    from metile_b200 import backends, synth

    w, s, b = synth.affine_weight(1, 64, 64)
    x = synth.activations(2, 1, 64)
    with pytest.raises(ValueError):
        backends.mlx_affine_qmv(x, w, s, b)  # CPU tensors: no CPU path
    with pytest.raises(TypeError):
        backends.mlx_affine_qmv(x.float(), w, s, b)
    with pytest.raises(ValueError):
        backends.mlx_affine_residual_qmv(x, w, s, b, x, group_size=32)
    with pytest.raises(ValueError):
        backends.mlx_affine_swiglu(x, w, s, None, w, s, b)
    with pytest.raises(ValueError):
        backends.MLXAffineWeight.from_mlx(w, s, b, bits=8)
    with pytest.raises(TypeError):
        backends.mlx_rms_norm(x, torch.ones(64), 1e-5)
