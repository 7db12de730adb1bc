"""Shared argument checks and pointer plumbing for the CUDA backends."""

from __future__ import annotations

import ctypes

import torch

from .. import _lib

PACKED_DTYPES = (torch.uint32, torch.int32)


def pointer(tensor):
    return None if tensor is None else ctypes.c_void_p(tensor.data_ptr())


# torch's own fast path to the raw handle of a device's current stream (what its compiled-kernel
# launchers use); `torch.cuda.current_stream()` builds a Stream object first and costs about six
# microseconds per call, a quarter of the host time of one operator call here.
_raw_current_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_pointer(device):
    if _raw_current_stream is not None:
        index = device.index if device.index is not None else torch.cuda.current_device()
        return ctypes.c_void_p(_raw_current_stream(index))
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def launch(function, device, *arguments):
    """Call a C-ABI entry point with `device` current and that device's current stream as last argument.

    The library takes its SM count, its per-device caches and its launches from the CURRENT device,
    so the tensors' device is made current around the call; a model on cuda:1 works while cuda:0 is
    current."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    if torch.cuda.current_device() == index:  # the common case: no device switch to pay for
        return function(*arguments, stream_pointer(device))
    with torch.cuda.device(device):
        return function(*arguments, stream_pointer(device))


def require_on_device(tensor, like, what, *, dtype=None, min_numel=None, contiguous=True):
    """Check a tensor whose raw pointer is about to cross the C ABI: a CUDA tensor on the same
    device as `like`, of the expected dtype, contiguous and at least `min_numel` elements long.
    A CPU tensor or one on another GPU would otherwise reach the kernel as a foreign pointer."""
    if tensor is None:
        return
    if not isinstance(tensor, torch.Tensor):
        raise TypeError(f"{what} must be a torch tensor")
    if not tensor.is_cuda or tensor.device != like.device:
        raise ValueError(f"{what} must live on the activations' CUDA device ({like.device}), got {tensor.device}")
    if dtype is not None and tensor.dtype != dtype:
        raise ValueError(f"{what} must be {dtype}, got {tensor.dtype}")
    if contiguous and not tensor.is_contiguous():
        raise ValueError(f"{what} must be contiguous")
    if min_numel is not None and tensor.numel() < min_numel:
        raise ValueError(f"{what} holds {tensor.numel()} elements, needs at least {min_numel}")


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
