"""Generate tests/golden/kat.npz: the reference's small test cases as known-answer vectors.

Run `python tests/golden/make_golden.py` from the repository root.

The reference (AndreSlavescu/meTile) stores no output arrays and its numeric tests compare
against MLX, which cannot be imported where this runs.  So the cases below re-create the
SHAPES and SEEDS of the reference's tests and record the outputs of oracle/affine.py:
  swiglu_1x64x64_s43      tests/test_mlx_backend.py:683-725
  swiglu_33x64x64_s49     tests/test_mlx_backend.py:1310-1368
  swiglu_{2,8}x256x128_s71 tests/test_mlx_backend.py:868-911
  residual_1x64x64_s54    tests/test_mlx_backend.py:927-971
  mlp_1x64_s55            tests/test_mlx_backend.py:974-1022
  qmm_{33,65,129}x64x64   tests/test_mlx_backend.py:1400-1459 (ragged prefill rows)
  qmm_1x64x64_s211        tests/test_affine_quantized.py:120-163 (same inputs as that test)
  add_rmsnorm_s29         tests/test_mlx_backend.py:3089-3118
  rmsnorm_s17             tests/test_mlx_backend.py:3065-3086
Weights: the reference quantises N(0,1) weights with mx.quantize; here q is uniform 0..15,
scale ~ U(0.002, 0.02), bias = -8*scale + N(0, 1e-3), all from numpy default_rng(seed).
bf16 arrays are stored as uint16 bit patterns.
"""

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import affine as A  # noqa: E402


def bits(x):
    return A.bf16_to_bits(x)


def main():
    out = {}

    def triple(rng, n, k):
        w, s, b = A.synth_affine(rng, n, k)
        return w, s, b

    def put_triple(prefix, t):
        out[prefix + "_w"], out[prefix + "_s"], out[prefix + "_b"] = t[0], bits(t[1]), bits(t[2])

    for name, rows, k, n, seed in (
        ("swiglu_1x64x64_s43", 1, 64, 64, 43),
        ("swiglu_33x64x64_s49", 33, 64, 64, 49),
        ("swiglu_2x256x128_s71", 2, 256, 128, 71),
        ("swiglu_8x256x128_s71", 8, 256, 128, 71),
    ):
        rng = np.random.default_rng(seed)
        x = A.bf16_round(rng.normal(size=(rows, k)))
        gate, up = triple(rng, n, k), triple(rng, n, k)
        out[name + "_x"] = bits(x)
        put_triple(name + "_gate", gate)
        put_triple(name + "_up", up)
        out[name + "_y"] = bits(A.swiglu_fused(x, gate, up))
        out[name + "_y_native"] = bits(A.swiglu_native(x, gate, up))

    rng = np.random.default_rng(54)
    x = A.bf16_round(rng.normal(size=(1, 64)))
    t = triple(rng, 64, 64)
    res = A.bf16_round(rng.normal(size=(1, 64)))
    out["residual_1x64x64_s54_x"], out["residual_1x64x64_s54_res"] = bits(x), bits(res)
    put_triple("residual_1x64x64_s54", t)
    out["residual_1x64x64_s54_y"] = bits(A.qmm(x, *t, residual=res))

    rng = np.random.default_rng(55)
    x = A.bf16_round(rng.normal(size=(1, 64)))
    gate, up, down = triple(rng, 64, 64), triple(rng, 64, 64), triple(rng, 64, 64)
    res = A.bf16_round(rng.normal(size=(1, 64)))
    out["mlp_1x64_s55_x"], out["mlp_1x64_s55_res"] = bits(x), bits(res)
    put_triple("mlp_1x64_s55_gate", gate)
    put_triple("mlp_1x64_s55_up", up)
    put_triple("mlp_1x64_s55_down", down)
    out["mlp_1x64_s55_y"] = bits(A.mlp(x, gate, up, down, res))

    for rows, seed in ((33, 53), (65, 59), (129, 59)):
        rng = np.random.default_rng(seed)
        x = A.bf16_round(rng.normal(size=(rows, 64)))
        t = triple(rng, 64, 64)
        name = f"qmm_{rows}x64x64"
        out[name + "_x"] = bits(x)
        put_triple(name, t)
        out[name + "_y"] = bits(A.qmm(x, *t))

    # Same inputs as the reference's numpy-only test (float16 there; rounded to bf16 here).
    rng = np.random.default_rng(211)
    x = A.bf16_round(rng.normal(size=(1, 64)))
    q = rng.integers(0, 16, size=(64, 64), dtype=np.uint8)
    s = A.bf16_round(rng.uniform(0.01, 0.2, size=(1, 64))).T.copy()
    b = A.bf16_round(rng.uniform(-0.5, 0.5, size=(1, 64))).T.copy()
    out["qmm_1x64x64_s211_x"] = bits(x)
    put_triple("qmm_1x64x64_s211", (A.pack_nibbles(q), s, b))
    out["qmm_1x64x64_s211_y"] = bits(A.qmm(x, A.pack_nibbles(q), s, b))

    rng = np.random.default_rng(29)
    x = A.bf16_round(rng.standard_normal((2, 1, 2048)))
    r = A.bf16_round(rng.standard_normal((2, 1, 2048)))
    w = A.bf16_round(rng.standard_normal((2048,)))
    total, norm = A.add_rmsnorm(x, r, w, 1e-5)
    out["add_rmsnorm_s29_x"], out["add_rmsnorm_s29_r"], out["add_rmsnorm_s29_w"] = bits(x), bits(r), bits(w)
    out["add_rmsnorm_s29_sum"], out["add_rmsnorm_s29_norm"] = bits(total), bits(norm)

    rng = np.random.default_rng(17)
    x = A.bf16_round(rng.standard_normal((2, 3, 2048)))
    w = A.bf16_round(rng.standard_normal((2048,)))
    out["rmsnorm_s17_x"], out["rmsnorm_s17_w"] = bits(x), bits(w)
    out["rmsnorm_s17_y"] = bits(A.rmsnorm(x, w, 1e-5))

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "kat.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
