"""CPU oracle for the MLX affine INT4 projection path.  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package imports this module.  It is the checker the tests,
the smoke entry and the benchmark's CPU-baseline leg compare the CUDA kernels against.

It restates, in numpy, the arithmetic of the reference project (AndreSlavescu/meTile),
citing the reference file:line each function follows.  The reference's own ground truth
for this path is a third-party package that is not part of the reference tree:
MLX (`mlx>=0.31` in the reference's pyproject.toml:24-30, measured with mlx 0.32.0),
`mx.quantized_matmul(x, W, scales, biases, transpose=True, group_size=64, bits=4,
mode="affine")`.  MLX cannot be installed or imported where this runs, and the
reference stores no output arrays, so:

  * what IS pinned by reference source and checked in tests/test_oracle.py: the packed
    layout (8 nibbles per uint32, least-significant nibble first), w = scale*q + bias,
    y = x @ w.T, the reference's only MLX-free numeric restatement
    (tests/test_affine_quantized.py:120-163, seed 211) and its fidelity-gate examples
    (tests/test_mlx_backend.py:1137-1146);
  * what is NOT pinned: MLX's internal accumulation order / dtype inside its CPU
    quantized_matmul.  For that boundary: PARITY UNPINNED.  The oracle accumulates in
    float64 so it sits inside any fp32-accumulating implementation's rounding envelope.

All arrays are numpy.  bf16 values travel as float32 arrays holding bf16-representable
numbers, or as uint16 bit patterns (`*_bits`).
"""

from __future__ import annotations

import numpy as np

GROUP_SIZE = 64
BITS = 4
VALUES_PER_WORD = 32 // BITS  # kernels/affine_qmv.py:25


# --------------------------------------------------------------------------- bf16 helpers
def bf16_round(values):
    """Round float32/float64 values to the nearest bf16 (ties to even); return float32."""
    as_f32 = np.ascontiguousarray(np.asarray(values, dtype=np.float32))
    bits = as_f32.view(np.uint32).astype(np.uint64)
    nan = np.isnan(as_f32)
    rounded = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    out = rounded.astype(np.uint32).view(np.float32).reshape(as_f32.shape)
    if nan.any():
        out = out.copy()
        out[nan] = np.nan
    return out


def bf16_round_f64(values):
    """Round float64 values to bf16 with a single rounding (no float32 step in between)."""
    v = np.asarray(values, dtype=np.float64)
    out = np.zeros(v.shape, dtype=np.float64)
    finite = np.isfinite(v) & (v != 0)
    mant, expo = np.frexp(np.where(finite, v, 1.0))  # v = mant * 2**expo, 0.5 <= |mant| < 1
    # bf16 keeps 8 significant bits; normal range only (inputs here are far from subnormal).
    scaled = np.ldexp(mant, 8)
    rounded = np.rint(scaled)  # ties to even
    out = np.where(finite, np.ldexp(rounded, expo - 8), v)
    return out.astype(np.float32)


def bf16_to_bits(values):
    """float32 array holding bf16-representable numbers -> uint16 bit patterns."""
    as_f32 = np.ascontiguousarray(np.asarray(values, dtype=np.float32))
    return (as_f32.view(np.uint32) >> 16).astype(np.uint16)


def bf16_from_bits(bits):
    """uint16 bf16 bit patterns -> float32."""
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# --------------------------------------------------------------------------- packing
def pack_nibbles(quantized):
    """q uint [N, K] (0..15) -> uint32 [N, K/8]; element 8j+e sits in bits [4e, 4e+4).

    Reference: kernels/affine_qmv.py:33-37,44-48 (word/element indexing) and
    metile/backends/mlx_quantized.py:768-769 (shifts 0,4,...,28).
    """
    q = np.asarray(quantized)
    if q.ndim != 2 or q.shape[1] % VALUES_PER_WORD:
        raise ValueError("expected [N, K] with K a multiple of 8")
    q = q.astype(np.uint32).reshape(q.shape[0], -1, VALUES_PER_WORD)
    shifts = np.arange(0, 32, BITS, dtype=np.uint32)
    return np.bitwise_or.reduce(q << shifts, axis=-1).astype(np.uint32)


def unpack_nibbles(packed):
    """uint32 [N, K/8] -> uint8 [N, K] (inverse of pack_nibbles)."""
    w = np.asarray(packed, dtype=np.uint32)
    shifts = np.arange(0, 32, BITS, dtype=np.uint32)
    q = (w[..., None] >> shifts) & 15
    return q.reshape(w.shape[0], -1).astype(np.uint8)


def repack_k_major(packed, scales, biases):
    """MLX layout -> the reference's K-major matrix-unit layout.

    Reference: metile/backends/mlx_quantized.py:754-774 (repack_mlx_affine_weight):
    nibbles transposed to K-major, two per byte with the even flat index in the low
    nibble; scales and biases transposed to [K/64, N].
    """
    q = unpack_nibbles(packed)
    flat = np.ascontiguousarray(q.T).reshape(-1)
    bytes_ = (flat[0::2] | (flat[1::2] << 4)).astype(np.uint8)
    return bytes_, np.ascontiguousarray(np.asarray(scales).T), np.ascontiguousarray(
        np.asarray(biases).T
    )


def dequantize(packed, scales, biases, *, group_size=GROUP_SIZE, weights="exact"):
    """w[n,k] = scales[n,k//g] * q[n,k] + biases[n,k//g]  (kernels/affine_qmv.py:41-51).

    weights="exact": float64, no rounding.
    weights="bf16":  each weight rounded once to bf16, RN(scale*q + bias) -- the form a
                     matrix-unit path feeds its MMA (the reference does the same in half:
                     metile/codegen/msl_emitter.py:1413-1418).
    """
    q = unpack_nibbles(packed).astype(np.float64)
    n, k = q.shape
    s = np.repeat(np.asarray(scales, dtype=np.float64), group_size, axis=1)
    b = np.repeat(np.asarray(biases, dtype=np.float64), group_size, axis=1)
    if s.shape != (n, k) or b.shape != (n, k):
        raise ValueError("scales/biases must be [N, K/group_size]")
    w = s * q + b
    if weights == "bf16":
        return bf16_round_f64(w).astype(np.float64)
    if weights != "exact":
        raise ValueError(weights)
    return w


# --------------------------------------------------------------------------- projections
def qmm(x, packed, scales, biases, *, residual=None, weights="exact", out="bf16",
        group_size=GROUP_SIZE):
    """y[r,n] = sum_k x[r,k] * w[n,k] (+ residual[r,n]), one rounding at the store.

    Reference: kernels/affine_qmv.py:30-53,86-91 (plain) and :124-131 (residual is added
    to the un-rounded sum, then stored once).  x may have leading batch dims.
    """
    x = np.asarray(x, dtype=np.float64)
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    w = dequantize(packed, scales, biases, group_size=group_size, weights=weights)
    y = x2 @ w.T
    if residual is not None:
        y = y + np.asarray(residual, dtype=np.float64).reshape(y.shape)
    y = y.reshape(*lead, w.shape[0])
    return _store(y, out)


def qmm_residual_native(x, packed, scales, biases, residual, **kw):
    """round(round(x@w.T) + residual): the two-op form of native MLX.

    Reference: metile/backends/mlx_quantized.py:845-855.
    """
    projected = qmm(x, packed, scales, biases, **kw).astype(np.float64)
    return bf16_round(projected + np.asarray(residual, dtype=np.float64))


def silu(values):
    v = np.asarray(values, dtype=np.float64)
    return v / (1.0 + np.exp(-v))


def swiglu_fused(x, gate, up, *, weights="exact", out="bf16"):
    """round( g/(1+exp(-g)) * u ) with g, u the un-rounded sums.

    Reference: kernels/affine_qmv.py:204-208.  `gate`/`up` are (packed, scales, biases).
    """
    g = qmm(x, *gate, weights=weights, out="f64")
    u = qmm(x, *up, weights=weights, out="f64")
    return _store(silu(g) * u, out)


def swiglu_native(x, gate, up, *, weights="exact"):
    """round( silu(round(g)) * round(u) ): MLX's op-by-op form.

    Reference: metile/backends/mlx_quantized.py:883-917.
    """
    g = qmm(x, *gate, weights=weights).astype(np.float64)
    u = qmm(x, *up, weights=weights).astype(np.float64)
    act = bf16_round(silu(g)).astype(np.float64)
    return bf16_round(act * u)


def mlp(x, gate, up, down, residual=None, *, weights="exact", out="bf16"):
    """down(swiglu(x)) + residual with the hidden activations materialised in bf16.

    Reference: metile/backends/mlx_quantized.py:1798,1829-1830 (the executor evaluates
    `hidden` in the storage dtype between the two kernels).
    """
    hidden = swiglu_fused(x, gate, up, weights=weights)
    return qmm(hidden, *down, residual=residual, weights=weights, out=out)


# --------------------------------------------------------------------------- norms
def add_rmsnorm(x, residual, weight, eps):
    """(Sum, Out) of the fused residual-add + RMSNorm.

    Reference: kernels/add_rmsnorm.py:7-25.  Sum = round(f32(x)+f32(res)); the sum of
    squares uses the UN-rounded f32 sums (:16); pass two reloads the ROUNDED Sum (:22).
    """
    xs = np.asarray(x, dtype=np.float64)
    rs = np.asarray(residual, dtype=np.float64)
    summed = np.asarray(xs + rs, dtype=np.float32).astype(np.float64)  # f32 add of two bf16
    total = bf16_round(summed)
    mean_square = np.mean(summed * summed, axis=-1, keepdims=True)
    inverse_rms = 1.0 / np.sqrt(mean_square + eps)
    out = total.astype(np.float64) * inverse_rms * np.asarray(weight, dtype=np.float64)
    return total, bf16_round(out)


def add_rmsnorm_native(x, residual, weight, eps):
    """Native two-op form: Sum as above, RMSNorm computed from the rounded Sum.

    Reference: metile/backends/mlx.py:536-538,827-828.
    """
    total = bf16_round(np.asarray(x, dtype=np.float64) + np.asarray(residual, dtype=np.float64))
    return total, rmsnorm(total, weight, eps)


def rmsnorm(x, weight, eps):
    """round( x * rsqrt(mean(x^2)+eps) * w ).  Reference: kernels/rmsnorm.py:5-26."""
    xs = np.asarray(x, dtype=np.float64)
    inverse_rms = 1.0 / np.sqrt(np.mean(xs * xs, axis=-1, keepdims=True) + eps)
    return bf16_round(xs * inverse_rms * np.asarray(weight, dtype=np.float64))


# --------------------------------------------------------------------------- dense rows
def _fma32(a, b, c):
    """float32 fused multiply-add (single rounding) for bf16-valued a, b."""
    return (np.asarray(a, np.float64) * np.asarray(b, np.float64)
            + np.asarray(c, np.float64)).astype(np.float32)


def dense_rows_f32(x, weight):
    """Exact fp32 result of the small-batch dense projection, before the bf16 store.

    Reference: metile/codegen/msl_emitter.py:1067-1120 -- lane l of a 32-lane group owns
    k = 128*b + 4*l .. +3 for b = 0,1,...; it accumulates in fp32 in ascending (b,
    component) order; lanes are combined by a shuffle-down tree with offsets 16, 8, 4,
    2, 1 and lane 0 holds the result.  Products of two bf16 values are exact in fp32, so
    each step is one rounding (fused multiply-add).  K must be a multiple of 128.
    """
    x = np.asarray(x, dtype=np.float32)
    w = np.asarray(weight, dtype=np.float32)
    rows, k = x.reshape(-1, x.shape[-1]).shape
    n = w.shape[0]
    if k % 128:
        raise ValueError("K must be a multiple of 128")
    x2 = x.reshape(rows, k)
    acc = np.zeros((rows, n, 32), dtype=np.float32)
    xb = x2.reshape(rows, k // 128, 32, 4)
    wb = w.reshape(n, k // 128, 32, 4)
    for block in range(k // 128):
        for comp in range(4):
            acc = _fma32(wb[None, :, block, :, comp], xb[:, None, block, :, comp], acc)
    for offset in (16, 8, 4, 2, 1):
        shifted = np.zeros_like(acc)
        shifted[..., : 32 - offset] = acc[..., offset:]
        # lanes >= 32 - offset read their own value in a real shuffle; they never feed lane 0.
        shifted[..., 32 - offset:] = acc[..., 32 - offset:]
        acc = (acc.astype(np.float32) + shifted.astype(np.float32)).astype(np.float32)
    return acc[..., 0].reshape(*x.shape[:-1], n)


def dense_rows(x, weight, residual=None):
    """bf16 store of dense_rows_f32, then the typed residual add.

    Reference: metile/codegen/msl_emitter.py:1111-1118: round to the storage dtype first,
    then add the residual in that dtype and round again.
    """
    projected = bf16_round(dense_rows_f32(x, weight))
    if residual is None:
        return projected
    return bf16_round(projected.astype(np.float64) + np.asarray(residual, dtype=np.float64))


def dense_swiglu(x, gate_weight, up_weight):
    """Typed SwiGLU epilogue of the dense small-batch path.

    Reference: metile/codegen/msl_emitter.py:1236-1251: left/right rounded to bf16,
    y = 1/(1+exp(|l|)), sigmoid = l<0 ? y : 1-y (rounded), activation = l*sigmoid
    (rounded), out = activation*right (rounded).
    """
    left = bf16_round(dense_rows_f32(x, gate_weight)).astype(np.float64)
    right = bf16_round(dense_rows_f32(x, up_weight)).astype(np.float64)
    y = 1.0 / (1.0 + np.exp(np.abs(left)))
    sigmoid = bf16_round(np.where(left < 0, y, 1.0 - y)).astype(np.float64)
    activation = bf16_round(left * sigmoid).astype(np.float64)
    return bf16_round(activation * right)


def matmul_act(a, b, activation):
    """C = act(A @ B) for the dense GEMM + activation entry points.

    Reference: kernels/mlp.py:28 (gelu: x/(1+exp(-1.702x))) and :55 (silu).
    """
    c = np.asarray(a, dtype=np.float64) @ np.asarray(b, dtype=np.float64)
    if activation == "silu":
        return bf16_round(c / (1.0 + np.exp(-c)))
    if activation == "gelu":
        return bf16_round(c / (1.0 + np.exp(-1.702 * c)))
    raise ValueError(activation)


# --------------------------------------------------------------------------- gates
def affine_swiglu_compatible(result, reference):
    """The reference's fidelity gate.  metile/backends/mlx_quantized.py:1256-1272."""
    result = np.asarray(result, dtype=np.float32)
    reference = np.asarray(reference, dtype=np.float32)
    if result.shape != reference.shape:
        return False
    difference = result - reference
    reference_rms = np.sqrt(np.mean(reference * reference))
    difference_rms = np.sqrt(np.mean(difference * difference))
    normalized_rms = difference_rms / max(reference_rms, 1e-6)
    normalized_peak = np.max(np.abs(difference)) / max(np.max(np.abs(reference)), 1e-6)
    finite = bool(np.all(np.isfinite(result)))
    return finite and normalized_rms <= 0.005 and normalized_peak <= 0.01


def accuracy_compatible(actual, reference):
    """max|d| <= 0.02 + 0.02*max|ref|.  metile/backends/mlx_affine.py:273-278."""
    actual = np.asarray(actual, dtype=np.float32)
    reference = np.asarray(reference, dtype=np.float32)
    return float(np.max(np.abs(actual - reference))) <= 0.02 + 0.02 * float(
        np.max(np.abs(reference))
    )


def bf16_ulp(values):
    """Spacing of bf16 numbers at |values| (8 significant bits): 2**(floor(log2|v|) - 7)."""
    v = np.abs(np.asarray(values, dtype=np.float64))
    _, expo = np.frexp(np.where(v > 0, v, 1.0))
    return np.where(v > 0, np.ldexp(1.0, expo - 1 - 7), 0.0)


def within_tolerance(actual, reference, rel=2e-3, store_ulps=1):
    """Scale-aware 2e-3 check on bf16 outputs.

    Every |y - y_ref| <= rel * max|y_ref| + store_ulps * ulp_bf16(y_ref).  The first term is the
    bound on the computation (fp32 accumulate, any summation order), in the form the
    reference's logits check uses (metile/compile.py:185-199: difference compared with
    tolerance * largest reference magnitude).  The second term is the bf16 store itself:
    bf16 keeps 8 significant bits, so its unit roundoff (2**-8 = 3.9e-3) is already larger
    than 2e-3, and two correctly rounded stores of nearly equal sums can differ by one ulp.
    Pass store_ulps=0 when comparing un-rounded values.  Returns (ok, worst_excess_ratio)
    where the ratio is max(|d| / bound).
    """
    actual = np.asarray(actual, dtype=np.float64)
    reference = np.asarray(reference, dtype=np.float64)
    peak = max(float(np.max(np.abs(reference))), 1e-30)
    bound = rel * peak + store_ulps * bf16_ulp(reference)
    ratio = float(np.max(np.abs(actual - reference) / bound))
    return bool(np.all(np.isfinite(actual))) and ratio <= 1.0, ratio


# --------------------------------------------------------------------------- generators
def synth_affine(rng, n, k, *, group_size=GROUP_SIZE):
    """Seeded synthetic INT4 weight: q uniform 0..15, scale ~ U(0.002, 0.02) in bf16,
    bias = -8*scale + N(0, 1e-3) in bf16.  Returns (packed u32 [N,K/8], scales, biases)."""
    q = rng.integers(0, 16, size=(n, k), dtype=np.uint8)
    scales = bf16_round(rng.uniform(0.002, 0.02, size=(n, k // group_size)))
    biases = bf16_round(-8.0 * scales + rng.normal(0.0, 1e-3, size=scales.shape))
    return pack_nibbles(q), scales, biases


def _store(y, out):
    if out == "bf16":
        return bf16_round_f64(y)
    if out == "f32":
        return np.asarray(y, dtype=np.float32)
    if out == "f64":
        return np.asarray(y, dtype=np.float64)
    raise ValueError(out)
