"""CPU oracle for decode attention, rotary embedding and the KV-cache append.  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package imports this module; the tests and the smoke entry compare the CUDA
kernels against it.

`attention_decode` restates the reference's online-softmax decode kernel
(kernels/attention.py:27-143 of AndreSlavescu/meTile): one query row per (batch, query head), grouped
query attention by integer division of the head index (:41-44), loads cast to float32 BEFORE the
scale multiplies the query (:58-62), `softmax(q.k * scale) @ v` accumulated in float32, one rounding
at the store.  The oracle accumulates in float64 and subtracts the row maximum, so it sits inside the
rounding envelope of any float32 online-softmax order (the reference's per-simdgroup partials
:64-96 and their merge :98-143 are one such order; a split over the KV range is another).

Its admission rule is the reference's `_supports_metile_decode`
(metile/integrations/mlx_lm.py:3558-3573): rank-4 [batch, heads, sequence, dim] arrays, query
length one, no mask, equal K/V shapes, query heads a multiple of KV heads, dim a multiple of 32.

Rotary embedding and the cache append are not meTile code: the reference leaves them to MLX-LM
(`nn.RoPE(dims, traditional=False, base=theta)` and `KVCache.update_and_fetch`, third-party
packages absent from the reference tree: `mlx-lm>=0.31` in pyproject.toml:24-30).  `rope` restates
the published half-split ("non-traditional") rotary form those models use; `kv_append` is a plain
indexed store.  PARITY UNPINNED for both: no reference test holds a rotary or cache vector.
"""

from __future__ import annotations

import numpy as np

from .affine import bf16_round


def supports_decode(queries_shape, keys_shape, values_shape):
    """The reference's shape gate for the decode kernel (mlx_lm.py:3558-3573)."""
    return (
        len(queries_shape) == len(keys_shape) == len(values_shape) == 4
        and queries_shape[2] == 1
        and tuple(keys_shape) == tuple(values_shape)
        and queries_shape[0] == keys_shape[0]
        and queries_shape[1] % keys_shape[1] == 0
        and queries_shape[-1] == keys_shape[-1]
        and queries_shape[-1] % 32 == 0
    )


def attention_decode(queries, keys, values, scale, lengths=None, out="bf16"):
    """queries [B, Hq, 1, D], keys / values [B, Hkv, N, D] (float32 arrays holding bf16 numbers) ->
    [B, Hq, 1, D].  `lengths[b]` limits batch entry b to its first tokens (None: all N)."""
    q = np.asarray(queries, dtype=np.float64)
    k = np.asarray(keys, dtype=np.float64)
    v = np.asarray(values, dtype=np.float64)
    if not supports_decode(q.shape, k.shape, v.shape):
        raise ValueError("decode attention expects [B,Hq,1,D] queries and matching [B,Hkv,N,D] keys/values")
    batch, q_heads, _, dim = q.shape
    kv_heads, tokens = k.shape[1], k.shape[2]
    group = q_heads // kv_heads
    result = np.zeros((batch, q_heads, 1, dim), dtype=np.float64)
    for b in range(batch):
        n = tokens if lengths is None else int(lengths[b])
        for h in range(q_heads):
            kv = h // group  # kernels/attention.py:43-44
            scores = (k[b, kv, :n] @ (q[b, h, 0] * scale))  # the query is scaled after the cast (:58-62)
            weights = np.exp(scores - scores.max())
            result[b, h, 0] = (weights @ v[b, kv, :n]) / weights.sum()
    return bf16_round(result) if out == "bf16" else result.astype(np.float32)


def rope(values, positions, theta, out="bf16"):
    """Half-split rotary embedding over the last axis: values [B, H, D] at positions [B].

    Pair (i, i + D/2) rotates by positions * theta**(-2i/D); computed in float64, one rounding."""
    x = np.asarray(values, dtype=np.float64)
    dim = x.shape[-1]
    half = dim // 2
    inverse = theta ** (-np.arange(0, dim, 2, dtype=np.float64) / dim)
    angles = np.asarray(positions, dtype=np.float64)[:, None, None] * inverse[None, None, :]
    cos, sin = np.cos(angles), np.sin(angles)
    first, second = x[..., :half], x[..., half:]
    rotated = np.concatenate([first * cos - second * sin, second * cos + first * sin], axis=-1)
    return bf16_round(rotated) if out == "bf16" else rotated.astype(np.float32)


def kv_append(key_cache, value_cache, new_keys, new_values, positions):
    """cache[b, h, positions[b], :] = new[b, h, :] for both caches, in place; returns the caches."""
    for b, position in enumerate(np.asarray(positions).tolist()):
        key_cache[b, :, position, :] = new_keys[b]
        value_cache[b, :, position, :] = new_values[b]
    return key_cache, value_cache
