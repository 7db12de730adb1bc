"""MLX-format affine INT4 projections on CUDA, behind the reference's operator names.

Reference surface reproduced (names, argument order, defaults, error behaviour):
  metile/backends/mlx_quantized.py:691  mlx_affine_qmv
  metile/backends/mlx_quantized.py:717  mlx_affine_swiglu_qmv
  metile/backends/mlx_quantized.py:1538 mlx_affine_residual_qmv
  metile/backends/mlx_quantized.py:1645 mlx_affine_swiglu
  metile/backends/mlx_quantized.py:1723 mlx_affine_swiglu_executor
  metile/backends/mlx_quantized.py:1770 mlx_affine_mlp_executor
  metile/backends/mlx_quantized.py:754  repack_mlx_affine_weight

Differences that are deliberate:
  * activations are bfloat16 torch CUDA tensors; packed weights keep the MLX layout unchanged;
  * there is no timing tournament: the kernel is chosen by row count (CUDA-core GEMV for one
    row, tcgen05 MMA above), so `autotune`, `block`, `outputs_per_simdgroup` and
    `decode_dtype` are accepted for call-site compatibility and ignored;
  * any number of rows is served from one read of the weights (the reference's scalar kernels
    re-read them per row and its tuned residual path hands multi-row inputs to native MLX,
    mlx_quantized.py:1569-1578);
  * unsupported formats raise; nothing is rerouted to another implementation.
"""

from __future__ import annotations

import contextlib
import ctypes
import threading

import torch

from .. import _lib
from ._common import (
    check_affine_triple,
    contiguous_2d,
    launch,
    library,
    pointer,
    require_cuda_bf16,
    require_on_device,
    rows_of,
)

_state = threading.local()
_dispatch_lock = threading.RLock()
_swiglu_dispatches = {}
_residual_dispatches = {}


def _flags():
    return getattr(_state, "flags", 0)


@contextlib.contextmanager
def batch_invariant(enabled=True):
    """Serve every row count from the tcgen05 kernel family, so that a row's output bits do not
    depend on whether it runs alone or in a batch of up to 128 (one accumulation order)."""
    previous = _flags()
    _state.flags = _lib.FLAG_FORCE_UMMA if enabled else 0
    try:
        yield
    finally:
        _state.flags = previous


@contextlib.contextmanager
def force_kernel(name):
    """Pin the kernel family: "gemv" (CUDA cores, up to 8 rows), "umma" (tcgen05), "mlp_fused" /
    "mlp_fused_mma" (the single-launch MLP on CUDA cores / on mma.sync; projections called on their
    own are unaffected) or None (the default dispatch by row count)."""
    table = {None: 0, "gemv": _lib.FLAG_FORCE_GEMV, "umma": _lib.FLAG_FORCE_UMMA,
             "mlp_fused": _lib.FLAG_MLP_FUSED, "mlp_fused_mma": _lib.FLAG_MLP_FUSED_MMA}
    if name not in table:
        raise ValueError(f"unknown kernel family {name!r}")
    previous = _flags()
    _state.flags = table[name]
    try:
        yield
    finally:
        _state.flags = previous


def _algorithm(rows, flags):
    if flags & _lib.FLAG_FORCE_GEMV:
        return "gemv"
    if flags & _lib.FLAG_FORCE_UMMA:
        return "umma"
    return "gemv" if rows <= 1 else "umma"


def _record(table, rows, input_features, output_features, dtype, group_size, bits, flags):
    key = (rows, input_features, output_features, str(dtype), group_size, bits)
    with _dispatch_lock:
        table[key] = _algorithm(rows, flags)


def _project(name, values, weight, scales, biases, residual, group_size, bits):
    require_cuda_bf16(values, name)
    output_features = check_affine_triple(name, values, weight, scales, biases, group_size, bits)
    expected_shape = (*values.shape[:-1], output_features)
    if residual is not None and (tuple(residual.shape) != expected_shape
                                 or residual.dtype != values.dtype):
        raise ValueError("residual must match the affine QMV output shape and dtype")
    require_on_device(residual, values, "residual", contiguous=False)
    x = contiguous_2d(values)
    res = None if residual is None else contiguous_2d(residual)
    out = torch.empty((x.shape[0], output_features), dtype=values.dtype, device=values.device)
    flags = _flags()
    code = launch(library().mt_affine_qmv, values.device, pointer(x), pointer(weight), pointer(scales),
                  pointer(biases), pointer(res), pointer(out), x.shape[0], x.shape[1], output_features,
                  group_size, bits, flags)
    _lib.check(code, name)
    return out.reshape(expected_shape), flags


def mlx_affine_qmv(values, weight, scales, biases, *, group_size=64, bits=4, block=32,
                   outputs_per_simdgroup=1, decode_dtype="f32"):
    """y = values @ dequant(weight)^T for any number of rows."""
    del block, outputs_per_simdgroup
    if decode_dtype not in ("f32", "f16"):
        raise ValueError("decode_dtype must be 'f32' or 'f16'")
    out, _ = _project("affine QMV", values, weight, scales, biases, None, group_size, bits)
    return out


def mlx_affine_residual_qmv(values, weight, scales, biases, residual, *, group_size=64, bits=4,
                            autotune=True):
    """y = values @ dequant(weight)^T + residual, the residual added before the one rounding."""
    del autotune
    out, flags = _project("affine residual QMV", values, weight, scales, biases, residual,
                          group_size, bits)
    _record(_residual_dispatches, rows_of(values), values.shape[-1], weight.shape[0], values.dtype,
            group_size, bits, flags)
    return out


def _swiglu(name, values, gate_weight, gate_scales, gate_biases, up_weight, up_scales, up_biases,
            group_size, bits):
    if not (bits == 4 and group_size == 64):
        raise ValueError(f"{name} requires 4-bit group-64 weights")
    if gate_biases is None or up_biases is None:
        raise ValueError(f"{name} requires affine quantization biases")
    require_cuda_bf16(values, name)
    if (
        values.dtype != gate_scales.dtype
        or values.dtype != gate_biases.dtype
        or gate_weight.shape != up_weight.shape
        or gate_scales.shape != up_scales.shape
        or gate_biases.shape != up_biases.shape
    ):
        raise ValueError(f"{name} requires matching gate/up weights and parameters")
    output_features = check_affine_triple(name, values, gate_weight, gate_scales, gate_biases,
                                          group_size, bits)
    check_affine_triple(name, values, up_weight, up_scales, up_biases, group_size, bits)
    x = contiguous_2d(values)
    out = torch.empty((x.shape[0], output_features), dtype=values.dtype, device=values.device)
    flags = _flags()
    code = launch(library().mt_affine_swiglu, values.device, pointer(x), pointer(gate_weight),
                  pointer(gate_scales), pointer(gate_biases), pointer(up_weight), pointer(up_scales),
                  pointer(up_biases), pointer(out), x.shape[0], x.shape[1], output_features, group_size,
                  bits, flags)
    _lib.check(code, name)
    _record(_swiglu_dispatches, x.shape[0], x.shape[1], output_features, values.dtype, group_size,
            bits, flags)
    return out.reshape(*values.shape[:-1], output_features)


def mlx_affine_swiglu_qmv(values, gate_weight, gate_scales, gate_biases, up_weight, up_scales,
                          up_biases, *, group_size=64, bits=4, block=32, outputs_per_simdgroup=1,
                          decode_dtype="f32"):
    """silu(values @ Wg^T) * (values @ Wu^T), SwiGLU applied to the un-rounded fp32 sums."""
    del block, outputs_per_simdgroup, decode_dtype
    return _swiglu("affine SwiGLU QMV", values, gate_weight, gate_scales, gate_biases, up_weight,
                   up_scales, up_biases, group_size, bits)


def mlx_affine_swiglu(values, gate_weight, gate_scales, gate_biases, up_weight, up_scales,
                      up_biases, *, group_size=64, bits=4, autotune=True):
    """Same computation as mlx_affine_swiglu_qmv; the reference's tuned dispatcher name."""
    del autotune
    return _swiglu("affine SwiGLU", values, gate_weight, gate_scales, gate_biases, up_weight,
                   up_scales, up_biases, group_size, bits)


def mlx_affine_swiglu_executor(sample_values, gate_weight, gate_scales, gate_biases, up_weight,
                               up_scales, up_biases, *, group_size=64, bits=4):
    """Validate once and return `execute(values)` bound to the weights."""
    mlx_affine_swiglu(sample_values, gate_weight, gate_scales, gate_biases, up_weight, up_scales,
                      up_biases, group_size=group_size, bits=bits)

    def execute(values):
        return _swiglu("affine SwiGLU", values, gate_weight, gate_scales, gate_biases, up_weight,
                       up_scales, up_biases, group_size, bits)

    return execute


def mlx_affine_mlp_executor(sample_values, gate_weight, gate_scales, gate_biases, up_weight,
                            up_scales, up_biases, down_weight, down_scales, down_biases,
                            sample_residual, *, group_size=64, bits=4):
    """Validate once and return `execute(values, residual)` = down(swiglu(values)) + residual.

    One C-ABI call (mt_affine_mlp) runs both kernels back to back on the current stream; the
    bf16 hidden activations live in a workspace the callable owns and grows on demand (calls of one
    executor on different streams would share it: give each stream its own executor).  Unlike the
    reference (metile/backends/mlx_quantized.py:1806-1820) any row count is accepted and no
    1-row call is needed first.
    """
    name = "affine MLP"
    require_cuda_bf16(sample_values, name)
    intermediate = check_affine_triple(name, sample_values, gate_weight, gate_scales, gate_biases,
                                       group_size, bits)
    check_affine_triple(name, sample_values, up_weight, up_scales, up_biases, group_size, bits)
    if gate_weight.shape != up_weight.shape:
        raise ValueError("affine MLP requires matching gate/up weights")
    hidden_features = sample_values.shape[-1]
    probe = torch.empty((1, intermediate), dtype=sample_values.dtype, device=sample_values.device)
    if check_affine_triple(name, probe, down_weight, down_scales, down_biases, group_size,
                           bits) != hidden_features:
        raise ValueError("affine MLP down projection must map back to the input width")
    if sample_residual is not None and (sample_residual.shape != sample_values.shape
                                        or sample_residual.dtype != sample_values.dtype):
        raise ValueError("residual must match the MLP output shape and dtype")
    lib = library()
    device = sample_values.device
    bound = (gate_weight, gate_scales, gate_biases, up_weight, up_scales, up_biases, down_weight,
             down_scales, down_biases)
    pointers = [pointer(t) for t in bound]

    workspace = {"hidden": None}  # grow-only scratch for the bf16 hidden activations, owned by the callable

    def execute(values, residual=None):
        if not isinstance(values, torch.Tensor) or values.dtype != torch.bfloat16 \
                or values.shape[-1] != hidden_features:
            raise ValueError("affine MLP executor received activations of a different layout")
        if not values.is_cuda or values.device != device:
            raise ValueError(f"affine MLP executor is bound to {device}; activations are on {values.device}")
        x = contiguous_2d(values)
        res = None
        if residual is not None:
            if residual.shape != values.shape or residual.dtype != values.dtype:
                raise ValueError("residual must match the MLP output shape and dtype")
            require_on_device(residual, values, "residual", contiguous=False)
            res = contiguous_2d(residual)
        rows = x.shape[0]
        hidden = workspace["hidden"]
        if hidden is None or hidden.numel() < rows * intermediate:
            hidden = workspace["hidden"] = torch.empty(rows * intermediate, dtype=torch.bfloat16, device=device)
        out = torch.empty((rows, hidden_features), dtype=torch.bfloat16, device=device)
        code = launch(lib.mt_affine_mlp, device, pointer(x), *pointers, pointer(res), pointer(hidden),
                      hidden.numel() * 2, pointer(out), rows, hidden_features, intermediate, group_size, bits,
                      _flags())
        _lib.check(code, name)
        return out.reshape(values.shape)

    # The raw pointers above stay valid only while the tensors live: the callable owns them.
    execute.weights = bound
    return execute


def mlx_affine_mlp_host_executor(max_rows, hidden_features, gate_weight, gate_scales, gate_biases, up_weight,
                                 up_scales, up_biases, down_weight, down_scales, down_biases, *,
                                 group_size=64, bits=4):
    """The fused MLP for activations that live in host memory.

    Returns `execute(values, residual, out)` on page-locked CPU bfloat16 tensors of up to `max_rows`
    rows: ONE C-ABI call (mt_affine_mlp_host) queues the host->device copies of the activations and
    the residual, the MLP kernels and the device->host copy of the result on the current stream;
    `out` is valid after `torch.cuda.current_stream().synchronize()`.  Device staging buffers and
    the hidden workspace are allocated once, here.  No counterpart in the reference (unified
    memory on Apple GPUs); the weights are the same MLX triples as for mlx_affine_mlp_executor.
    """
    name = "affine MLP (host buffers)"
    device = gate_weight.device
    probe = torch.empty((1, hidden_features), dtype=torch.bfloat16, device=device)
    intermediate = check_affine_triple(name, probe, gate_weight, gate_scales, gate_biases, group_size, bits)
    check_affine_triple(name, probe, up_weight, up_scales, up_biases, group_size, bits)
    if gate_weight.shape != up_weight.shape:
        raise ValueError("affine MLP requires matching gate/up weights")
    probe_down = torch.empty((1, intermediate), dtype=torch.bfloat16, device=device)
    if check_affine_triple(name, probe_down, down_weight, down_scales, down_biases, group_size,
                           bits) != hidden_features:
        raise ValueError("affine MLP down projection must map back to the input width")
    lib = library()
    bound = (gate_weight, gate_scales, gate_biases, up_weight, up_scales, up_biases, down_weight,
             down_scales, down_biases)
    pointers = [pointer(t) for t in bound]
    staging = torch.empty((3, max_rows, hidden_features), dtype=torch.bfloat16, device=device)
    workspace = torch.empty((max_rows, intermediate), dtype=torch.bfloat16, device=device)
    stage_pointers = [ctypes.c_void_p(staging[i].data_ptr()) for i in range(3)]
    row_bytes = hidden_features * 2

    stage_base = staging[0].data_ptr()
    workspace_pointer, workspace_bytes = pointer(workspace), workspace.numel() * 2
    entry = lib.mt_affine_mlp_host

    def execute(values, residual, out):
        for tensor in (values, residual, out):
            if tensor is None:
                continue
            if tensor.is_cuda or tensor.dtype != torch.bfloat16 or not tensor.is_contiguous():
                raise ValueError("host executor expects contiguous CPU bfloat16 tensors")
            if tensor.shape[-1] != hidden_features or tensor.shape != values.shape:
                raise ValueError("host executor received tensors of a different layout")
        rows = values.numel() // hidden_features
        if rows > max_rows:
            raise ValueError(f"host executor was sized for {max_rows} rows, got {rows}")
        # The residual staging area starts right after the rows in use, so that a residual that
        # follows the activations in host memory travels in the same copy.
        residual_stage = ctypes.c_void_p(stage_base + rows * row_bytes) if rows < max_rows else stage_pointers[1]
        flags = _flags()
        values_address = values.data_ptr()
        residual_address = None if residual is None else residual.data_ptr()
        if (residual_address is not None and residual_address == values_address + rows * row_bytes
                and residual.untyped_storage().data_ptr() == values.untyped_storage().data_ptr()):
            flags |= _lib.FLAG_HOST_PAIR  # two views of one page-locked buffer: one copy moves both
        code = launch(entry, device, values_address, residual_address, out.data_ptr(), stage_pointers[0], residual_stage,
                      stage_pointers[2], *pointers, workspace_pointer, workspace_bytes, rows, hidden_features,
                      intermediate, group_size, bits, flags)
        _lib.check(code, name)
        return out

    execute.weights = bound
    execute.buffers = (staging, workspace)
    return execute


def repack_mlx_affine_weight(weight, scales, biases):
    """MLX output-major layout -> the reference's K-major layout (two nibbles per byte, even flat
    index in the low nibble; scales and biases transposed).  Provided for callers that hold
    K-major consumers; the CUDA kernels here read the MLX layout directly and never need it."""
    if biases is None:
        raise ValueError("native affine QMV requires affine biases")
    if weight.ndim != 2 or scales.ndim != 2 or biases.shape != scales.shape:
        raise ValueError("expected packed weight and matching two-dimensional parameters")
    words = weight.to(torch.int64) & 0xFFFFFFFF
    shifts = torch.arange(0, 32, 4, device=weight.device, dtype=torch.int64)
    quantized = ((words[..., None] >> shifts) & 15).to(torch.uint8)
    quantized = quantized.reshape(weight.shape[0], weight.shape[1] * 8).t().reshape(-1)
    packed = quantized[0::2] | (quantized[1::2] << 4)
    return packed, scales.t().contiguous(), biases.t().contiguous()


def _dispatch_rows(table):
    with _dispatch_lock:
        items = sorted(table.items())
    return tuple(
        {
            "rows": key[0],
            "input_features": key[1],
            "output_features": key[2],
            "dtype": key[3],
            "group_size": key[4],
            "bits": key[5],
            "algorithm": algorithm,
            "implementation": "metile_b200",
        }
        for key, algorithm in items
    )


def mlx_affine_swiglu_dispatches():
    """Which kernel family served each SwiGLU shape in this process."""
    return _dispatch_rows(_swiglu_dispatches)


def mlx_affine_residual_qmv_dispatches():
    """Which kernel family served each residual projection shape in this process."""
    return _dispatch_rows(_residual_dispatches)


__all__ = [
    "batch_invariant",
    "force_kernel",
    "mlx_affine_mlp_host_executor",
    "mlx_affine_mlp_executor",
    "mlx_affine_qmv",
    "mlx_affine_residual_qmv",
    "mlx_affine_residual_qmv_dispatches",
    "mlx_affine_swiglu",
    "mlx_affine_swiglu_dispatches",
    "mlx_affine_swiglu_executor",
    "mlx_affine_swiglu_qmv",
    "repack_mlx_affine_weight",
]
