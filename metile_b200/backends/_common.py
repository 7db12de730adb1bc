"""Shared argument checks and pointer plumbing for the CUDA backends."""

from __future__ import annotations

import ctypes

import torch

from .. import _lib

PACKED_DTYPES = (torch.uint32, torch.int32)


def pointer(tensor):
    return None if tensor is None else ctypes.c_void_p(tensor.data_ptr())


def stream_pointer(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def require_cuda_bf16(values, what):
    if not isinstance(values, torch.Tensor):
        raise TypeError(f"{what} expects torch tensors")
    if values.dtype != torch.bfloat16:
        raise TypeError(f"{what} supports bfloat16 activations only, got {values.dtype}")
    if not values.is_cuda:
        raise ValueError(f"{what} expects CUDA tensors; there is no CPU path")


def rows_of(values):
    return values.numel() // values.shape[-1] if values.shape[-1] else 0


def contiguous_2d(values):
    return values.reshape(-1, values.shape[-1]).contiguous()


def check_affine_triple(name, values, weight, scales, biases, group_size, bits):
    """The reference's shape / dtype contract (metile/backends/mlx_quantized.py:1550-1565)."""
    if group_size != 64 or bits != 4:
        raise ValueError(f"{name} requires 4-bit weights with group size 64")
    if biases is None:
        raise ValueError(f"{name} requires affine quantization biases")
    input_features = values.shape[-1]
    if weight.ndim != 2 or weight.dtype not in PACKED_DTYPES:
        raise ValueError(f"{name} expects a two-dimensional uint32 packed weight")
    output_features = weight.shape[0]
    parameter_shape = (output_features, input_features // group_size)
    if (
        weight.shape[1] * 32 // bits != input_features
        or tuple(scales.shape) != parameter_shape
        or tuple(biases.shape) != parameter_shape
    ):
        raise ValueError(f"{name} received incompatible quantization parameters")
    if scales.dtype != values.dtype or biases.dtype != values.dtype:
        raise ValueError(f"{name} parameters must match the input dtype")
    for tensor in (weight, scales, biases):
        if not tensor.is_cuda or tensor.device != values.device:
            raise ValueError(f"{name} expects every tensor on the activation's CUDA device")
        if not tensor.is_contiguous():
            raise ValueError(f"{name} expects contiguous packed weights and parameters")
    return output_features


def library():
    return _lib.load()
