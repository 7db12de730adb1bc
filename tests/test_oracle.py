"""CPU tests that pin the oracle: layout, the reference's MLX-free restatement, its fidelity
gate examples, the C port, and the committed known-answer vectors."""

import os

import numpy as np
import pytest

from oracle import affine as A
from oracle import cport

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "kat.npz")


def test_pack_unpack_round_trip_and_nibble_order():
    rng = np.random.default_rng(0)
    q = rng.integers(0, 16, size=(5, 64), dtype=np.uint8)
    packed = A.pack_nibbles(q)
    assert packed.dtype == np.uint32 and packed.shape == (5, 8)
    assert (A.unpack_nibbles(packed) == q).all()
    # kernels/affine_qmv.py:44-48: element e of a word is (packed >> 4e) & 15.
    one = A.pack_nibbles(np.array([[1, 2, 3, 4, 5, 6, 7, 8]], dtype=np.uint8))
    assert int(one[0, 0]) == 0x87654321


def test_reference_numpy_restatement_seed_211():
    """tests/test_affine_quantized.py:120-163 of the reference, computed as it computes it."""
    random = np.random.default_rng(211)
    activations = random.normal(size=(1, 64)).astype(np.float16)
    quantized = random.integers(0, 16, size=(64, 64), dtype=np.uint8)
    scales = random.uniform(0.01, 0.2, size=(1, 64)).astype(np.float16)
    biases = random.uniform(-0.5, 0.5, size=(1, 64)).astype(np.float16)
    expected_weight = quantized.astype(np.float32) * scales.T.astype(np.float32) + biases.T.astype(
        np.float32)
    expected = (activations.astype(np.float32) @ expected_weight.T).astype(np.float16)
    mine = A.qmm(activations.astype(np.float32), A.pack_nibbles(quantized),
                 scales.T.astype(np.float32), biases.T.astype(np.float32), out="f32")
    np.testing.assert_allclose(mine, expected.astype(np.float32), rtol=3e-2, atol=3e-2)
    # The oracle is float64 inside, so it agrees with the float32 restatement far more tightly.
    np.testing.assert_allclose(mine, activations.astype(np.float32) @ expected_weight.T, rtol=1e-4,
                               atol=1e-4)
    # K-major repack of the same weights (mlx_quantized.py:768-772, test lines 131-132).
    k_major = np.ascontiguousarray(quantized.T).reshape(-1)
    packed_ref = np.ascontiguousarray(k_major[0::2] | (k_major[1::2] << 4), dtype=np.uint8)
    packed_mine, s_t, b_t = A.repack_k_major(A.pack_nibbles(quantized), scales.T, biases.T)
    assert (packed_mine == packed_ref).all() and s_t.shape == (1, 64) and b_t.shape == (1, 64)


def test_fidelity_gate_examples():
    """tests/test_mlx_backend.py:1137-1146 of the reference."""
    reference = np.array([0.0, 1000.0, -2000.0], dtype=np.float32)
    assert A.affine_swiglu_compatible(np.array([0.2, 1001.0, -1998.0], dtype=np.float32), reference)
    assert not A.affine_swiglu_compatible(np.array([0.0, 1015.0, -1960.0], dtype=np.float32), reference)
    assert A.accuracy_compatible(reference + 0.01, reference)


def test_oracle_reproduces_golden_vectors():
    kat = np.load(GOLDEN)

    def t(prefix):
        return kat[prefix + "_w"], A.bf16_from_bits(kat[prefix + "_s"]), A.bf16_from_bits(kat[prefix + "_b"])

    for name in ("swiglu_1x64x64_s43", "swiglu_33x64x64_s49", "swiglu_2x256x128_s71",
                 "swiglu_8x256x128_s71"):
        x = A.bf16_from_bits(kat[name + "_x"])
        y = A.swiglu_fused(x, t(name + "_gate"), t(name + "_up"))
        assert (A.bf16_to_bits(y) == kat[name + "_y"]).all(), name
    for rows in (33, 65, 129):
        name = f"qmm_{rows}x64x64"
        y = A.qmm(A.bf16_from_bits(kat[name + "_x"]), *t(name))
        assert (A.bf16_to_bits(y) == kat[name + "_y"]).all()
    total, norm = A.add_rmsnorm(A.bf16_from_bits(kat["add_rmsnorm_s29_x"]),
                                A.bf16_from_bits(kat["add_rmsnorm_s29_r"]),
                                A.bf16_from_bits(kat["add_rmsnorm_s29_w"]), 1e-5)
    assert (A.bf16_to_bits(total) == kat["add_rmsnorm_s29_sum"]).all()
    assert (A.bf16_to_bits(norm) == kat["add_rmsnorm_s29_norm"]).all()


def test_add_rmsnorm_sum_is_the_dtype_add():
    """tests/test_mlx_backend.py:3108-3111: Sum equals x + residual computed in the storage dtype."""
    import torch

    rng = np.random.default_rng(29)
    x = A.bf16_round(rng.standard_normal((2, 1, 2048)))
    r = A.bf16_round(rng.standard_normal((2, 1, 2048)))
    w = A.bf16_round(rng.standard_normal((2048,)))
    total, norm = A.add_rmsnorm(x, r, w, 1e-5)
    expected = (torch.from_numpy(x).bfloat16() + torch.from_numpy(r).bfloat16()).float().numpy()
    assert (total == expected).all()
    native_total, native_norm = A.add_rmsnorm_native(x, r, w, 1e-5)
    assert (native_total == total).all()
    np.testing.assert_allclose(norm, native_norm, rtol=4e-2, atol=4e-2)


def test_rmsnorm_matches_numpy_cases():
    """tests/test_rmsnorm.py:8-89: shapes incl. a non-power-of-two width, zero input, unit weights."""
    rng = np.random.default_rng(1)
    for rows, cols in ((32, 64), (64, 128), (64, 300), (1, 512), (1, 2048)):
        x = A.bf16_round(rng.standard_normal((rows, cols)))
        w = np.ones(cols, dtype=np.float32)
        ref = x / np.sqrt(np.mean(x.astype(np.float64) ** 2, axis=-1, keepdims=True) + 1e-5)
        np.testing.assert_allclose(A.rmsnorm(x, w, 1e-5), ref, rtol=1e-2, atol=1e-2)
    assert (A.rmsnorm(np.zeros((4, 64), np.float32), np.ones(64, np.float32), 1e-5) == 0).all()


def test_c_port_agrees_with_numpy_oracle():
    rng = np.random.default_rng(7)
    m, h, inter = 5, 128, 256
    gate, up, down = A.synth_affine(rng, inter, h), A.synth_affine(rng, inter, h), A.synth_affine(rng, h, inter)
    x = A.bf16_round(rng.normal(size=(m, h)))
    res = A.bf16_round(rng.normal(size=(m, h)))

    def b(t):
        return t[0], A.bf16_to_bits(t[1]), A.bf16_to_bits(t[2])

    y = A.bf16_from_bits(cport.qmm(A.bf16_to_bits(x), *b(gate)))
    assert A.within_tolerance(y, A.qmm(x, *gate))[0]
    s = A.bf16_from_bits(cport.swiglu(A.bf16_to_bits(x), b(gate), b(up)))
    assert A.within_tolerance(s, A.swiglu_fused(x, gate, up))[0]
    full = A.bf16_from_bits(cport.mlp(A.bf16_to_bits(x), b(gate), b(up), b(down), A.bf16_to_bits(res)))
    assert A.within_tolerance(full, A.mlp(x, gate, up, down, res))[0]
    w = A.bf16_round(1 + 0.02 * rng.normal(size=h))
    total, norm = cport.add_rmsnorm(A.bf16_to_bits(x), A.bf16_to_bits(res), A.bf16_to_bits(w), 1e-6)
    o_total, o_norm = A.add_rmsnorm(x, res, w, 1e-6)
    assert (total == A.bf16_to_bits(o_total)).all()
    assert A.within_tolerance(A.bf16_from_bits(norm), o_norm)[0]
    assert cport.num_threads() >= 1


def test_bf16_weight_variant_is_close_to_exact():
    rng = np.random.default_rng(3)
    t = A.synth_affine(rng, 64, 512)
    x = A.bf16_round(rng.normal(size=(4, 512)))
    assert A.within_tolerance(A.qmm(x, *t, weights="bf16"), A.qmm(x, *t, weights="exact"))[0]
    # Un-rounded sums: the bf16 weight rounding alone stays under 2e-3 of the output peak.
    ok, ratio = A.within_tolerance(A.qmm(x, *t, weights="bf16", out="f64"),
                                   A.qmm(x, *t, weights="exact", out="f64"), store_ulps=0)
    assert ok and ratio < 1.0


def test_dense_rows_order_and_invariance():
    rng = np.random.default_rng(4177)
    w = A.bf16_round(rng.normal(size=(16, 256)) * 0.02)
    x = A.bf16_round(rng.normal(size=(4, 256)))
    full = A.dense_rows_f32(x, w)
    for row in range(4):
        assert (A.dense_rows_f32(x[row:row + 1], w) == full[row:row + 1]).all()
    np.testing.assert_allclose(full, x.astype(np.float64) @ w.astype(np.float64).T, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("bad", [(63, 64), (64, 60)])
def test_pack_rejects_bad_shapes(bad):
    with pytest.raises(ValueError):
        A.pack_nibbles(np.zeros((bad[0], bad[1] + 1), dtype=np.uint8)[:, :-1][:, : bad[1] - 3])
