"""Residual add + RMSNorm and RMSNorm on CUDA, behind the reference's operator names.

Reference: metile/backends/mlx.py:786-830 (mlx_add_rms_norm) and :748-783 (mlx_rms_norm).
The reference runs a timing tournament between block sizes and native MLX; here there is one
hand-written kernel per op, so `autotune` is accepted and ignored.

Also here: decode attention (metile/backends/mlx.py:718-747, mlx_attention_decode) and the rotary
embedding + in-place KV-cache append that precedes it in a decoder block.
"""

from __future__ import annotations

import ctypes

import torch

from .. import _lib
from ._common import launch, library, pointer, require_cuda_bf16, require_on_device, rows_of


def mlx_rms_norm(values, weight, eps, *, autotune=True):
    """RMSNorm over the last axis: bf16(x * rsqrt(mean(x^2) + eps) * w)."""
    del autotune
    if values.ndim < 1 or weight.ndim != 1 or values.shape[-1] != weight.shape[0]:
        raise ValueError("meTile RMSNorm requires a matching one-dimensional weight")
    if values.dtype != weight.dtype:
        raise TypeError("meTile RMSNorm requires matching input and weight dtypes")
    require_cuda_bf16(values, "meTile RMSNorm")
    require_on_device(weight, values, "RMSNorm weight", contiguous=False)
    x = values.contiguous()
    w = weight.contiguous()
    out = torch.empty_like(x)
    if x.numel() == 0:
        return out
    code = launch(library().mt_rmsnorm, x.device, pointer(x), pointer(w), pointer(out), rows_of(x), x.shape[-1],
                  ctypes.c_float(float(eps)))
    _lib.check(code, "mlx_rms_norm")
    return out


def mlx_add_rms_norm(values, residual, weight, eps, *, autotune=True):
    """Fused residual add + RMSNorm; returns (summed, normalized)."""
    del autotune
    if values.shape != residual.shape or values.dtype != residual.dtype:
        raise ValueError("meTile fused add/RMSNorm requires matching residual inputs")
    if values.ndim < 1 or weight.ndim != 1 or values.shape[-1] != weight.shape[0]:
        raise ValueError("meTile fused add/RMSNorm requires a matching RMSNorm weight")
    if values.dtype != weight.dtype:
        raise TypeError("meTile fused add/RMSNorm requires matching input and weight dtypes")
    require_cuda_bf16(values, "meTile fused add/RMSNorm")
    require_on_device(residual, values, "residual", contiguous=False)
    require_on_device(weight, values, "RMSNorm weight", contiguous=False)
    x = values.contiguous()
    r = residual.contiguous()
    w = weight.contiguous()
    summed = torch.empty_like(x)
    normalized = torch.empty_like(x)
    if x.numel() == 0:
        return summed, normalized
    code = launch(library().mt_add_rmsnorm, x.device, pointer(x), pointer(r), pointer(w), pointer(summed),
                  pointer(normalized), rows_of(x), x.shape[-1], ctypes.c_float(float(eps)))
    _lib.check(code, "mlx_add_rms_norm")
    return summed, normalized


def supports_attention_decode(query, key, value, mask=None):
    """None when the decode-attention kernel can serve this call, else the reason it cannot.

    The reference's admission rule (metile/integrations/mlx_lm.py:3558-3573): rank-4
    [batch, heads, sequence, dim] arrays, a query of length one, no mask, equal key / value shapes,
    query heads a multiple of the KV heads, matching dtypes; narrowed to what the CUDA kernel serves
    (bfloat16 on one CUDA device, head dim 64 or 128, at most 8 query heads per KV head)."""
    if mask is not None:
        return "a mask was given"
    if query.ndim != 4 or key.ndim != 4 or value.ndim != 4:
        return "query, key and value must be rank-four arrays"
    if query.shape[2] != 1:
        return "the query is not a single decode row"
    if key.shape != value.shape or query.shape[0] != key.shape[0]:
        return "batch or key/value shapes do not match"
    if query.shape[1] % key.shape[1] or query.shape[1] // key.shape[1] > 8:
        return "query heads must be 1 to 8 times the key/value heads"
    if query.shape[-1] != key.shape[-1] or query.shape[-1] not in (64, 128):
        return "head dimension must be 64 or 128 and match"
    if not (query.dtype == key.dtype == value.dtype == torch.bfloat16):
        return "query, key and value must be bfloat16"
    if not query.is_cuda or key.device != query.device or value.device != query.device:
        return "query, key and value must share one CUDA device"
    if key.shape[2] < 1:
        return "the cache is empty"
    return None


def _cache_layout(tensor):
    """(base tensor pointer, capacity) of a [B, H, N, D] cache or of a view of its first N tokens."""
    batch, heads, tokens, dim = tensor.shape
    strides = tensor.stride()
    if strides[3] != 1 or strides[2] != dim or strides[1] % dim or strides[0] != heads * strides[1]:
        return None
    capacity = strides[1] // dim
    return capacity if capacity >= tokens else None


def mlx_attention_decode(query, key, value, *, scale, autotune=True, lengths=None):
    """softmax(scale * q k^T) v for one query row per sequence and head.

    query [B, Hq, 1, D]; key, value [B, Hkv, N, D] -- contiguous, or the first-N-tokens view of a
    larger in-place cache [B, Hkv, capacity, D] (no copy is made either way).  `lengths` (int32 [B] on
    the device) limits sequence b to its first lengths[b] tokens.  Returns [B, Hq, 1, D]."""
    del autotune
    if query.ndim != 4 or key.ndim != 4 or value.ndim != 4:
        raise ValueError("meTile attention expects rank-four query, key, and value arrays")
    if query.shape[2] != 1:
        raise ValueError("meTile attention currently supports decode queries of length one")
    if key.shape != value.shape or query.shape[0] != key.shape[0]:
        raise ValueError("meTile attention requires matching batch and key/value shapes")
    if query.shape[1] % key.shape[1]:
        raise ValueError("key/value heads must divide query heads")
    if query.dtype != key.dtype or query.dtype != value.dtype:
        raise TypeError("meTile attention requires matching input dtypes")
    require_cuda_bf16(query, "meTile attention")
    reason = supports_attention_decode(query, key, value)
    if reason is not None:
        raise ValueError(f"meTile attention: {reason}")
    capacity = _cache_layout(key)
    if capacity is None or _cache_layout(value) != capacity:
        key, value = key.contiguous(), value.contiguous()
        capacity = key.shape[2]
    batch, q_heads, _, dim = query.shape
    kv_heads, tokens = key.shape[1], key.shape[2]
    q = query.reshape(batch, q_heads, dim).contiguous()
    out = torch.empty_like(q)
    lib = library()
    needed = lib.mt_attention_decode_workspace_bytes(batch, q_heads, tokens, dim)
    workspace = torch.empty(max(needed, 16) // 4, dtype=torch.float32, device=query.device)
    if lengths is not None:
        require_on_device(lengths, query, "lengths", dtype=torch.int32, min_numel=batch)
    code = launch(lib.mt_attention_decode, query.device, pointer(q), pointer(key), pointer(value), pointer(lengths),
                  pointer(out), pointer(workspace), workspace.numel() * 4, batch, q_heads, kv_heads, tokens, capacity,
                  dim, ctypes.c_float(float(scale)))
    _lib.check(code, "mlx_attention_decode")
    return out.reshape(batch, q_heads, 1, dim)


def rope_kv_append(query, key, value, positions, key_cache, value_cache, *, theta):
    """Rotate the new query and key rows and append key and value to the caches, in place.

    query [B, Hq, D], key / value [B, Hkv, D] -- dense, or three views into the rows of one fused
    q|k|v projection [B, (Hq + 2 Hkv) D] (no copy is made); positions int32 [B] (device): the row of
    each sequence's cache [B, Hkv, capacity, D] that receives the new token.  Returns the rotated
    query as a dense [B, Hq, D] tensor."""
    require_cuda_bf16(query, "rope_kv_append")
    batch, q_heads, dim = query.shape
    kv_heads, capacity = key_cache.shape[1], key_cache.shape[2]
    if key.shape != (batch, kv_heads, dim) or value.shape != key.shape:
        raise ValueError("rope_kv_append expects key and value rows of shape [batch, kv_heads, head_dim]")
    if key_cache.shape != (batch, kv_heads, capacity, dim) or value_cache.shape != key_cache.shape:
        raise ValueError("rope_kv_append expects caches of shape [batch, kv_heads, capacity, head_dim]")
    for label, tensor in (("key cache", key_cache), ("value cache", value_cache)):
        require_on_device(tensor, query, label, dtype=torch.bfloat16)
    for label, tensor in (("key", key), ("value", value)):
        require_on_device(tensor, query, label, dtype=torch.bfloat16, contiguous=False)
    require_on_device(positions, query, "positions", dtype=torch.int32, min_numel=batch)

    def head_major(tensor):
        return tensor.stride(2) == 1 and tensor.stride(1) == dim

    # The kernel reads sequence b of q, k and v at b * row_stride from their base pointers: true of
    # views into one fused q|k|v projection; dense arrays of different widths are staged in one buffer.
    common = head_major(query) and head_major(key) and head_major(value) and (
        batch == 1 or query.stride(0) == key.stride(0) == value.stride(0))
    if not common:
        fused = torch.cat([query.reshape(batch, -1), key.reshape(batch, -1), value.reshape(batch, -1)], dim=1)
        query = fused[:, :q_heads * dim].view(batch, q_heads, dim)
        key = fused[:, q_heads * dim:(q_heads + kv_heads) * dim].view(batch, kv_heads, dim)
        value = fused[:, (q_heads + kv_heads) * dim:].view(batch, kv_heads, dim)
    row_stride = query.stride(0) if batch > 1 else (q_heads + 2 * kv_heads) * dim
    out = torch.empty((batch, q_heads, dim), dtype=torch.bfloat16, device=query.device)
    code = launch(library().mt_rope_kv_append, query.device, pointer(query), pointer(key), pointer(value),
                  ctypes.c_longlong(int(row_stride)), pointer(positions), pointer(out), pointer(key_cache),
                  pointer(value_cache), batch, q_heads, kv_heads, capacity, dim, ctypes.c_float(float(theta)))
    _lib.check(code, "rope_kv_append")
    return out
