"""GPU parity tests: the CUDA kernels (called through the C ABI via the operator entry points)
against the CPU oracle, the committed known-answer vectors, and size-independent properties.

Tolerance (see oracle.affine.within_tolerance): every |y - y_ref| <= 2e-3 * max|y_ref| plus one
bf16 ulp for the store.  The CUDA-core GEMV keeps weights exact in fp32 and is compared with the
exact-weight oracle.  The tcgen05 path rounds each dequantised weight once to bf16 before the
MMA (as the reference's matrix-unit path does in half), so it is compared with the oracle's
weights="bf16" variant at the same bound, and with the exact-weight oracle through the
reference's own acceptance gate (RMS <= 0.5 %, peak <= 1 %).
"""

import os

import numpy as np
import pytest
import torch

from metile_b200 import _lib, backends as B, synth
from metile_b200.kernels import add_rmsnorm as k_add_rmsnorm
from metile_b200.kernels import affine_qmv as k_qmv
from metile_b200.kernels import mlp as k_mlp
from metile_b200.kernels import rmsnorm as k_rmsnorm
from oracle import affine as A
from tests.helpers import assert_bit_equal, assert_within, f32, triple_np

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "kat.npz")
FAMILIES = ("gemv", "umma")
MAX_ROWS = {"gemv": 8, "umma": 128}


def oracle_weights(family):
    return "exact" if family == "gemv" else "bf16"


def bf16_tensor(bits, device):
    return torch.from_numpy(np.ascontiguousarray(bits)).view(torch.bfloat16).to(device)


def golden_triple(kat, prefix, device):
    return (torch.from_numpy(kat[prefix + "_w"]).to(device), bf16_tensor(kat[prefix + "_s"], device),
            bf16_tensor(kat[prefix + "_b"], device))


def golden_triple_np(kat, prefix):
    return kat[prefix + "_w"], A.bf16_from_bits(kat[prefix + "_s"]), A.bf16_from_bits(kat[prefix + "_b"])


@pytest.fixture(autouse=True)
def no_device_wait_gave_up(cuda_device):
    assert _lib.load().mt_device_check() == 0
    yield
    ok, words = _lib.device_status()
    assert ok, f"a bounded device-side wait gave up: {[hex(w) for w in words]}"


# ----------------------------------------------------------------------------- golden vectors
@pytest.mark.parametrize("family", FAMILIES)
@pytest.mark.parametrize("name", ["swiglu_1x64x64_s43", "swiglu_33x64x64_s49", "swiglu_2x256x128_s71",
                                  "swiglu_8x256x128_s71"])
def test_golden_swiglu(cuda_device, family, name):
    kat = np.load(GOLDEN)
    x = bf16_tensor(kat[name + "_x"], cuda_device)
    if x.shape[0] > MAX_ROWS[family]:
        pytest.skip(f"the {family} family serves up to {MAX_ROWS[family]} rows")
    gate, up = golden_triple(kat, name + "_gate", cuda_device), golden_triple(kat, name + "_up", cuda_device)
    with B.force_kernel(family):
        y = B.mlx_affine_swiglu(x, *gate, *up)
    reference = A.swiglu_fused(f32(x), golden_triple_np(kat, name + "_gate"), golden_triple_np(kat, name + "_up"),
                               weights=oracle_weights(family))
    assert_within(y, reference, what=f"{family} {name}")
    # The stored vector (exact weights) and MLX's op-by-op form, at the reference's own tolerance.
    np.testing.assert_allclose(f32(y), A.bf16_from_bits(kat[name + "_y"]), rtol=3e-2, atol=3e-2)
    np.testing.assert_allclose(f32(y), A.bf16_from_bits(kat[name + "_y_native"]), rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("family", FAMILIES)
def test_golden_residual_and_mlp(cuda_device, family):
    kat = np.load(GOLDEN)
    name = "residual_1x64x64_s54"
    x, res = bf16_tensor(kat[name + "_x"], cuda_device), bf16_tensor(kat[name + "_res"], cuda_device)
    with B.force_kernel(family):
        y = B.mlx_affine_residual_qmv(x, *golden_triple(kat, name, cuda_device), res)
    assert_within(y, A.qmm(f32(x), *golden_triple_np(kat, name), residual=f32(res), weights=oracle_weights(family)))
    np.testing.assert_allclose(f32(y), A.bf16_from_bits(kat[name + "_y"]), rtol=3e-2, atol=3e-2)

    name = "mlp_1x64_s55"
    x, res = bf16_tensor(kat[name + "_x"], cuda_device), bf16_tensor(kat[name + "_res"], cuda_device)
    triples = [golden_triple(kat, f"{name}_{part}", cuda_device) for part in ("gate", "up", "down")]
    execute = B.mlx_affine_mlp_executor(x, *triples[0], *triples[1], *triples[2], res)
    with B.force_kernel(family):
        y = execute(x, res)
    np.testing.assert_allclose(f32(y), A.bf16_from_bits(kat[name + "_y"]), rtol=3e-2, atol=3e-2)
    triples_np = [golden_triple_np(kat, f"{name}_{part}") for part in ("gate", "up", "down")]
    assert_within(y, A.mlp(f32(x), *triples_np, f32(res), weights=oracle_weights(family)), rel=3e-3)


@pytest.mark.parametrize("rows", [33, 65, 129])
def test_golden_ragged_prefill_rows(cuda_device, rows):
    """Ragged row counts (33 / 65 / 129) as in the reference's prefill tests; 129 spans two launches."""
    kat = np.load(GOLDEN)
    name = f"qmm_{rows}x64x64"
    x = bf16_tensor(kat[name + "_x"], cuda_device)
    y = B.mlx_affine_qmv(x, *golden_triple(kat, name, cuda_device))
    assert y.shape == (rows, 64)
    assert_within(y, A.qmm(f32(x), *golden_triple_np(kat, name), weights="bf16"))
    np.testing.assert_allclose(f32(y), A.bf16_from_bits(kat[name + "_y"]), rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("family", FAMILIES)
def test_golden_numpy_only_case_seed_211(cuda_device, family):
    kat = np.load(GOLDEN)
    name = "qmm_1x64x64_s211"
    x = bf16_tensor(kat[name + "_x"], cuda_device)
    with B.force_kernel(family):
        y = B.mlx_affine_qmv(x, *golden_triple(kat, name, cuda_device))
    np.testing.assert_allclose(f32(y), A.bf16_from_bits(kat[name + "_y"]), rtol=3e-2, atol=3e-2)
    assert_within(y, A.qmm(f32(x), *golden_triple_np(kat, name), weights=oracle_weights(family)))


def test_golden_norms(cuda_device):
    kat = np.load(GOLDEN)
    x, r, w = (bf16_tensor(kat["add_rmsnorm_s29_" + k], cuda_device) for k in ("x", "r", "w"))
    total, norm = B.mlx_add_rms_norm(x, r, w, 1e-5)
    assert total.shape == x.shape == norm.shape
    assert (f32(total) == A.bf16_from_bits(kat["add_rmsnorm_s29_sum"])).all()  # exact, as the reference asserts
    assert_bit_equal(total, x + r, "Sum vs the dtype add")
    np.testing.assert_allclose(f32(norm), A.bf16_from_bits(kat["add_rmsnorm_s29_norm"]), rtol=4e-2, atol=4e-2)
    assert_within(norm, A.bf16_from_bits(kat["add_rmsnorm_s29_norm"]))
    x, w = bf16_tensor(kat["rmsnorm_s17_x"], cuda_device), bf16_tensor(kat["rmsnorm_s17_w"], cuda_device)
    y = B.mlx_rms_norm(x, w, 1e-5)
    np.testing.assert_allclose(f32(y), A.bf16_from_bits(kat["rmsnorm_s17_y"]), rtol=4e-2, atol=4e-2)
    assert_within(y, A.bf16_from_bits(kat["rmsnorm_s17_y"]))


# ----------------------------------------------------------------------------- seeded shapes
SHAPES = [(64, 64), (256, 128), (512, 200), (1536, 1024), (2048, 512), (8192, 256), (8960, 384)]


@pytest.mark.parametrize("family", FAMILIES)
@pytest.mark.parametrize("k,n", SHAPES)
def test_projection_variants_against_oracle(cuda_device, family, k, n):
    rows_list = {"gemv": (1, 2, 5, 8)}.get(family, (1, 3, 16, 17, 64, 100, 128))
    gate, up = synth.affine_weight(10, n, k, cuda_device), synth.affine_weight(11, n, k, cuda_device)
    gate_np, up_np = triple_np(gate), triple_np(up)
    weights = oracle_weights(family)
    for rows in rows_list:
        x = synth.activations(20 + rows, rows, k, cuda_device)
        res = synth.activations(40 + rows, rows, n, cuda_device)
        with B.force_kernel(family):
            y = B.mlx_affine_qmv(x, *gate)
            y_res = B.mlx_affine_residual_qmv(x, *gate, res)
            y_swi = B.mlx_affine_swiglu(x, *gate, *up)
        assert_within(y, A.qmm(f32(x), *gate_np, weights=weights), what=f"{family} qmv {rows}x{k}x{n}")
        assert_within(y_res, A.qmm(f32(x), *gate_np, residual=f32(res), weights=weights),
                      what=f"{family} residual {rows}x{k}x{n}")
        assert_within(y_swi, A.swiglu_fused(f32(x), gate_np, up_np, weights=weights),
                      what=f"{family} swiglu {rows}x{k}x{n}")
        # Against exact weights: the reference's acceptance gate for a kernel it would keep.
        assert A.affine_swiglu_compatible(f32(y_swi), A.swiglu_fused(f32(x), gate_np, up_np))
        assert A.accuracy_compatible(f32(y), A.qmm(f32(x), *gate_np))


def test_config0_gemv_1536_8960(cuda_device):
    """The single projection of a Qwen2.5-1.5B MLP: M=1, K=1536, N=8960."""
    k, n = 1536, 8960
    weight = synth.affine_weight(0, n, k, cuda_device)
    x = synth.activations(1, 1, k, cuda_device)
    weight_np = triple_np(weight)
    y = B.mlx_affine_qmv(x, *weight)
    assert y.shape == (1, n) and y.dtype == torch.bfloat16
    assert_within(y, A.qmm(f32(x), *weight_np), what="1536 -> 8960 projection (default dispatch)")
    with B.batch_invariant():
        y_mma = B.mlx_affine_qmv(x, *weight)
    assert_within(y_mma, A.qmm(f32(x), *weight_np, weights="bf16"), what="1536 -> 8960 projection (tcgen05)")
    # Second checker: the C port (fp32 accumulate).
    from oracle import cport

    y_c = A.bf16_from_bits(cport.qmm(synth.to_numpy_bits(x), weight_np[0], A.bf16_to_bits(weight_np[1]),
                                     A.bf16_to_bits(weight_np[2])))
    assert_within(y, y_c, what="1536 -> 8960 projection vs C port")


@pytest.mark.parametrize("rows", [1, 2, 4, 8, 16, 32, 128])
def test_config1_fused_mlp_llama_1b(cuda_device, rows):
    """The Llama-3.2-1B MLP: hidden 2048, intermediate 8192, full sizes, through mt_affine_mlp."""
    hidden, inter = 2048, 8192
    gate, up, down = synth.mlp_weights(100, hidden, inter, cuda_device)
    x = synth.activations(5, rows, hidden, cuda_device)
    res = synth.activations(6, rows, hidden, cuda_device)
    execute = B.mlx_affine_mlp_executor(x, *gate, *up, *down, res)
    y = execute(x, res)
    assert y.shape == (rows, hidden)
    from oracle import cport

    bits = [(t[0].cpu().numpy(), synth.to_numpy_bits(t[1]), synth.to_numpy_bits(t[2])) for t in (gate, up, down)]
    y_c = A.bf16_from_bits(cport.mlp(synth.to_numpy_bits(x), *bits, synth.to_numpy_bits(res)))
    # Two fp32-accumulating implementations with a bf16 hidden layer in between: 4e-3 of the peak.
    assert_within(y, y_c, rel=3e-3, what=f"MLP M={rows} vs C port")
    assert A.affine_swiglu_compatible(f32(y), y_c)
    # Linearity in the residual: mlp(x, r) - mlp(x, 0) == r up to the two bf16 stores.
    y0 = execute(x, torch.zeros_like(res))
    delta = f32(y) - f32(y0) - f32(res)
    assert np.abs(delta).max() <= 2 * A.bf16_ulp(np.abs(f32(y)).max() + np.abs(f32(res)).max())


@pytest.mark.parametrize("hidden,inter", [(2048, 8192), (1024, 2048), (1024, 1024), (2048, 4096), (4096, 2048)])
def test_single_launch_mlp_up_to_four_rows(cuda_device, hidden, inter):
    """The single-launch MLP kernel (one to four activation rows): exact weights, compared with the
    oracle at the MLP tolerance; a row's bits do not depend on how many rows share the launch; the
    default dispatch uses it for one row; repeated back-to-back launches (programmatic
    dependent launch between them) give the same bits."""
    gate, up, down = synth.mlp_weights(300, hidden, inter, cuda_device)
    triples_np = [triple_np(t) for t in (gate, up, down)]
    x = synth.activations(5, 4, hidden, cuda_device)
    res = synth.activations(6, 4, hidden, cuda_device)
    execute = B.mlx_affine_mlp_executor(x, *gate, *up, *down, res)
    library = _lib.load()
    with B.force_kernel("mlp_fused"):
        full = execute(x, res)
        again = [execute(x, res) for _ in range(4)]
        for rows in (1, 2, 3):
            assert_bit_equal(execute(x[:rows], res[:rows]), full[:rows], f"{rows} rows alone vs in a batch of 4")
        assert_bit_equal(execute(x[3:4], res[3:4]), full[3:4], "last row alone")
    assert_within(full, A.mlp(f32(x), *triples_np, f32(res)), rel=3e-3, what=f"single-launch MLP {hidden}x{inter}")
    for other in again:
        assert_bit_equal(other, full, "repeat launch")
    assert library.mt_affine_mlp_launches(1, hidden, inter, 0) == 1
    assert_bit_equal(execute(x[:1], res[:1]), full[:1], "default dispatch at one row is this kernel")
    assert library.mt_affine_mlp_launches(4, hidden, inter, _lib.FLAG_MLP_FUSED) == 1
    # Without a residual, and against the two-kernel path: two approximations of the same MLP (exact
    # weights here, bf16-rounded weights there), each within 3e-3 of the oracle, so within 6e-3 of each other.
    no_residual = B.mlx_affine_mlp_executor(x, *gate, *up, *down, None)
    with B.force_kernel("mlp_fused"):
        y_plain = no_residual(x, None)
    assert_within(y_plain, A.mlp(f32(x), *triples_np, None), rel=3e-3, what="single-launch MLP, no residual")
    with B.force_kernel("umma"):
        y_two = execute(x, res)
    assert_within(full, f32(y_two), rel=6e-3, what="single-launch vs two-kernel path")


@pytest.mark.parametrize("hidden,inter", [(2048, 8192), (1024, 2048), (1024, 1024), (2048, 4096), (512, 1536)])
def test_single_launch_mlp_on_warp_mma_up_to_eight_rows(cuda_device, hidden, inter):
    """The warp-MMA variant of the single-launch MLP (default for two to eight rows): exact weights,
    oracle at the MLP tolerance, rows bit-identical alone or in a batch of eight, repeatable."""
    gate, up, down = synth.mlp_weights(320, hidden, inter, cuda_device)
    triples_np = [triple_np(t) for t in (gate, up, down)]
    x = synth.activations(5, 8, hidden, cuda_device)
    res = synth.activations(6, 8, hidden, cuda_device)
    execute = B.mlx_affine_mlp_executor(x, *gate, *up, *down, res)
    library = _lib.load()
    with B.force_kernel("mlp_fused_mma"):
        full = execute(x, res)
        assert_bit_equal(execute(x, res), full, "repeat launch")
        for rows in (1, 3, 4, 5, 7):
            assert_bit_equal(execute(x[:rows], res[:rows]), full[:rows], f"{rows} rows alone vs in a batch of 8")
        assert_bit_equal(execute(x[7:8], res[7:8]), full[7:8], "last row alone")
        y_plain = B.mlx_affine_mlp_executor(x, *gate, *up, *down, None)(x, None)
    assert_within(full, A.mlp(f32(x), *triples_np, f32(res)), rel=3e-3, what=f"warp-MMA MLP {hidden}x{inter}")
    assert_within(y_plain, A.mlp(f32(x), *triples_np, None), rel=3e-3, what="warp-MMA MLP, no residual")
    for rows in (2, 3, 4, 8):
        assert library.mt_affine_mlp_launches(rows, hidden, inter, 0) == 1
        assert_bit_equal(execute(x[:rows], res[:rows]), full[:rows], "default dispatch is the warp-MMA kernel")
    assert library.mt_affine_mlp_launches(9, hidden, inter, 0) == 2
    assert library.mt_affine_mlp_launches(9, hidden, inter, _lib.FLAG_MLP_FUSED_MMA) == 2


def test_single_launch_mlp_refuses_what_it_does_not_serve(cuda_device):
    gate, up, down = synth.mlp_weights(301, 2048, 8192, cuda_device)
    x = synth.activations(5, 5, 2048, cuda_device)
    execute = B.mlx_affine_mlp_executor(x, *gate, *up, *down, x)
    with B.force_kernel("mlp_fused"):
        with pytest.raises(ValueError):
            execute(x, x)  # five rows
    x9 = synth.activations(5, 9, 2048, cuda_device)
    with B.force_kernel("mlp_fused_mma"):
        with pytest.raises(ValueError):
            B.mlx_affine_mlp_executor(x9, *gate, *up, *down, x9)(x9, x9)  # nine rows
    gate, up, down = synth.mlp_weights(302, 1536, 1024, cuda_device)
    x = synth.activations(5, 1, 1536, cuda_device)
    execute = B.mlx_affine_mlp_executor(x, *gate, *up, *down, x)
    with B.force_kernel("mlp_fused"):
        with pytest.raises(ValueError):
            execute(x, x)  # width that is not a whole number of 1024-column sets
    assert _lib.load().mt_affine_mlp_launches(1, 1536, 1024, 0) == 2
    assert_within(execute(x, x), A.mlp(f32(x), *[triple_np(t) for t in (gate, up, down)], f32(x)), rel=3e-3)


# ----------------------------------------------------------------------------- batch invariance
@pytest.mark.parametrize("k,n", [(2048, 512), (1536, 1024), (8192, 256)])
def test_batch_invariance_bit_exact_1_to_128(cuda_device, k, n):
    """Each row's output is bit-identical alone or inside a batch of up to 128 (one kernel family)."""
    gate, up = synth.affine_weight(10, n, k, cuda_device), synth.affine_weight(11, n, k, cuda_device)
    x = synth.activations(99, 128, k, cuda_device)
    res = synth.activations(98, 128, n, cuda_device)
    with B.batch_invariant():
        alone_swi = torch.cat([B.mlx_affine_swiglu(x[i:i + 1], *gate, *up) for i in range(128)])
        alone_res = torch.cat([B.mlx_affine_residual_qmv(x[i:i + 1], *gate, res[i:i + 1]) for i in range(128)])
        for rows in (2, 4, 8, 16, 17, 32, 64, 100, 128):
            assert_bit_equal(B.mlx_affine_swiglu(x[:rows], *gate, *up), alone_swi[:rows], f"swiglu M={rows}")
            assert_bit_equal(B.mlx_affine_residual_qmv(x[:rows], *gate, res[:rows]), alone_res[:rows],
                             f"residual M={rows}")
        # A row does not depend on WHICH other rows share its batch either.
        shuffled = torch.randperm(128, generator=torch.Generator().manual_seed(3)).to(cuda_device)
        assert_bit_equal(B.mlx_affine_swiglu(x[shuffled], *gate, *up), alone_swi[shuffled], "shuffled batch")


@pytest.mark.parametrize("family", ["gemv", "umma"])
def test_batch_invariance_within_each_family(cuda_device, family):
    k, n = 2048, 512
    gate, up = synth.affine_weight(10, n, k, cuda_device), synth.affine_weight(11, n, k, cuda_device)
    top = MAX_ROWS[family]
    x = synth.activations(99, top, k, cuda_device)
    with B.force_kernel(family):
        alone = torch.cat([B.mlx_affine_swiglu(x[i:i + 1], *gate, *up) for i in range(top)])
        for rows in {"gemv": (2, 3, 4, 8)}.get(family, (16, 33, 128)):
            assert_bit_equal(B.mlx_affine_swiglu(x[:rows], *gate, *up), alone[:rows], f"{family} M={rows}")


def test_mlp_batch_invariance_and_repeatability(cuda_device):
    hidden, inter = 2048, 8192
    gate, up, down = synth.mlp_weights(100, hidden, inter, cuda_device)
    x = synth.activations(5, 128, hidden, cuda_device)
    res = synth.activations(6, 128, hidden, cuda_device)
    execute = B.mlx_affine_mlp_executor(x[:1], *gate, *up, *down, res[:1])
    with B.batch_invariant():
        full = execute(x, res)
        assert_bit_equal(execute(x, res), full, "same call twice")
        for rows in (1, 8, 16, 32):
            assert_bit_equal(execute(x[:rows], res[:rows]), full[:rows], f"MLP M={rows}")
        assert_bit_equal(execute(x[77:78], res[77:78]), full[77:78], "row 77 alone")


# ----------------------------------------------------------------------------- norms, dense
@pytest.mark.parametrize("rows,width", [(1, 1536), (16, 1536), (512, 1536), (2, 2048), (3, 300), (7, 64), (4, 8192)])
def test_add_rmsnorm_and_rmsnorm(cuda_device, rows, width):
    x, r = synth.activations(1, rows, width, cuda_device), synth.activations(2, rows, width, cuda_device)
    w = synth.norm_weight(3, width, cuda_device)
    total, norm = B.mlx_add_rms_norm(x, r, w, 1e-6)
    o_total, o_norm = A.add_rmsnorm(f32(x), f32(r), f32(w), 1e-6)
    assert (f32(total) == o_total).all()
    assert_within(norm, o_norm, what="add_rmsnorm")
    assert_within(B.mlx_rms_norm(x, w, 1e-6), A.rmsnorm(f32(x), f32(w), 1e-6), what="rmsnorm")
    # Row independence: any row alone gives the same bits.
    alone_total, alone_norm = B.mlx_add_rms_norm(x[rows - 1:], r[rows - 1:], w, 1e-6)
    assert_bit_equal(alone_norm, norm[rows - 1:], "add_rmsnorm row alone")
    # Kernel-level signatures.
    total2, norm2 = torch.empty_like(x), torch.empty_like(x)
    k_add_rmsnorm.add_rmsnorm(x, r, w, total2, norm2, width, 1e-6, 256)
    assert_bit_equal(total2, total)
    assert_bit_equal(norm2, norm)
    out = torch.empty_like(x)
    k_rmsnorm.rmsnorm(x, w, out, width, 1e-6, 256)
    assert_bit_equal(out, B.mlx_rms_norm(x, w, 1e-6))


def test_norm_edge_cases(cuda_device):
    zeros = torch.zeros((4, 64), dtype=torch.bfloat16, device=cuda_device)
    ones = torch.ones((64,), dtype=torch.bfloat16, device=cuda_device)
    assert float(B.mlx_rms_norm(zeros, ones, 1e-5).abs().max()) == 0.0
    empty = torch.zeros((0, 64), dtype=torch.bfloat16, device=cuda_device)
    total, norm = B.mlx_add_rms_norm(empty, empty, ones, 1e-5)
    assert total.shape == (0, 64) and norm.shape == (0, 64)
    rank3 = synth.activations(1, 6, 2048, cuda_device).reshape(2, 3, 2048)
    w = synth.norm_weight(3, 2048, cuda_device)
    assert B.mlx_rms_norm(rank3, w, 1e-5).shape == (2, 3, 2048)
    with pytest.raises(ValueError):
        B.mlx_add_rms_norm(rank3, rank3[:1], w, 1e-5)
    with pytest.raises(TypeError):
        B.mlx_rms_norm(rank3, w.float(), 1e-5)


@pytest.mark.parametrize("k,n", [(256, 128), (256, 256), (1536, 8960)])
def test_dense_rows_bit_exact_and_batch_invariant(cuda_device, k, n):
    """Dense bf16 small-batch projection (K=1536, N=8960): per-row outputs bit-identical."""
    w = synth.dense_weight(5, n, k, cuda_device)
    g = synth.dense_weight(6, n, k, cuda_device)
    x = synth.activations(7, 128, k, cuda_device)
    r = synth.activations(8, 128, n, cuda_device)
    rows_list = (1, 2, 4, 8, 16, 32, 128)
    alone = torch.cat([B.mlx_dense_residual_qmv(x[i:i + 1], w, r[i:i + 1]) for i in range(32)])
    for rows in rows_list:
        y = B.mlx_dense_residual_qmv(x[:rows], w, r[:rows])
        assert_bit_equal(y[:32], alone[:min(rows, 32)], f"dense residual M={rows}")
    small = 8
    reference = A.dense_rows(f32(x[:small]), f32(w), f32(r[:small]))
    assert (f32(B.mlx_dense_residual_qmv(x[:small], w, r[:small])) == reference).all()
    swi = B.mlx_dense_swiglu(x[:small], g, w)
    assert_within(swi, A.dense_swiglu(f32(x[:small]), f32(g), f32(w)), what="dense swiglu")
    alone_swi = torch.cat([B.mlx_dense_swiglu(x[i:i + 1], g, w) for i in range(small)])
    assert_bit_equal(swi, alone_swi, "dense swiglu rows alone")
    # rank-3 activations, as tests/test_mlx_backend.py:348-406 of the reference.
    rank3 = x[:6].reshape(2, 3, k)
    assert_bit_equal(B.mlx_dense_residual_qmv(rank3, w).reshape(6, n), B.mlx_dense_residual_qmv(x[:6], w))


def test_matmul_silu_and_gelu(cuda_device):
    m, n, k = 16, 200, 96
    a = synth.activations(1, m, k, cuda_device, std=0.5)
    b = synth.activations(2, k, n, cuda_device, std=0.5)
    c = torch.empty((m, n), dtype=torch.bfloat16, device=cuda_device)
    k_mlp.matmul_silu(a, b, c, m, n, k)
    assert_within(c, A.matmul_act(f32(a), f32(b), "silu"), what="matmul_silu")
    k_mlp.matmul_gelu(a, b, c, m, n, k)
    assert_within(c, A.matmul_act(f32(a), f32(b), "gelu"), what="matmul_gelu")
    with pytest.raises(ValueError):
        big = torch.empty((200, k), dtype=torch.bfloat16, device=cuda_device)
        k_mlp.matmul_silu(big, b, torch.empty((200, n), dtype=torch.bfloat16, device=cuda_device), 200, n, k)


# ----------------------------------------------------------------------------- API surface
def test_kernel_level_entry_points_and_weight_object(cuda_device):
    k, n, rows = 256, 128, 4
    gate, up, down = synth.mlp_weights(7, k, n, cuda_device)
    x = synth.activations(1, rows, k, cuda_device)
    res = synth.activations(2, rows, n, cuda_device)
    out = torch.empty((rows, n), dtype=torch.bfloat16, device=cuda_device)
    k_qmv.affine_qmv(x, *gate, out, k, n, 64, 4, 32, 1, False)
    assert_bit_equal(out, B.mlx_affine_qmv(x, *gate))
    k_qmv.affine_residual_qmv(x, *gate, res, out, k, n, 64, 4, 64, 2, False)
    assert_bit_equal(out, B.mlx_affine_residual_qmv(x, *gate, res))
    k_qmv.affine_swiglu_qmv(x, *gate, *up, out, k, n, 64, 4, 32, 1, False)
    assert_bit_equal(out, B.mlx_affine_swiglu_qmv(x, *gate, *up))
    scratch = torch.empty_like(out)
    k_qmv.affine_swiglu_scratch_qmv(x, *gate, *up, scratch, k, n, 64, 4, 32, 1, False)
    assert_bit_equal(scratch, out)  # reference: scratch == register-fused bitwise
    weight = B.MLXAffineWeight.from_mlx(*gate)
    assert weight.shape == (k, n)
    assert_bit_equal(B.mlx_affine_matmul(x, weight), B.mlx_affine_qmv(x, *gate))
    hidden = torch.empty((rows, n), dtype=torch.bfloat16, device=cuda_device)
    y = torch.empty((rows, k), dtype=torch.bfloat16, device=cuda_device)
    xr = synth.activations(3, rows, k, cuda_device)
    k_mlp.affine_swiglu_mlp(x, *gate, *up, *down, xr, hidden, y)
    execute = B.mlx_affine_mlp_executor(x, *gate, *up, *down, xr)
    assert_bit_equal(y, execute(x, xr))
    assert_bit_equal(hidden, B.mlx_affine_swiglu(x, *gate, *up))
    swiglu_execute = B.mlx_affine_swiglu_executor(x, *gate, *up)
    assert_bit_equal(swiglu_execute(x), hidden)
    rank3 = x.reshape(2, 2, k)
    assert B.mlx_affine_qmv(rank3, *gate).shape == (2, 2, n)
    assert any(d["algorithm"] in ("gemv", "umma") for d in B.mlx_affine_swiglu_dispatches())
    packed, s_t, b_t = B.repack_mlx_affine_weight(*gate)
    ref_packed, _, _ = A.repack_k_major(*triple_np(gate))
    assert (packed.cpu().numpy() == ref_packed).all() and s_t.shape == (k // 64, n)


def test_errors_raise_and_nothing_falls_back(cuda_device):
    k, n = 128, 64
    w, s, b = synth.affine_weight(1, n, k, cuda_device)
    x = synth.activations(2, 2, k, cuda_device)
    with pytest.raises(ValueError):
        B.mlx_affine_qmv(x, w, s, b, group_size=32)
    with pytest.raises(ValueError):
        B.mlx_affine_qmv(x, w, s, b, bits=8)
    with pytest.raises(ValueError):
        B.mlx_affine_residual_qmv(x, w, s, b, x)  # residual of the wrong width
    with pytest.raises(ValueError):
        B.mlx_affine_qmv(x[:, :64], w, s, b)
    with pytest.raises(ValueError):
        B.mlx_affine_swiglu(x, w, s, b, w[:32], s[:32], b[:32])
    with pytest.raises(TypeError):
        B.mlx_affine_qmv(x.half(), w, s, b)
    with pytest.raises(ValueError):
        with B.force_kernel("gemv"):
            B.mlx_affine_qmv(synth.activations(2, 9, k, cuda_device), w, s, b)  # GEMV serves <= 8 rows
    empty = B.mlx_affine_qmv(x[:0], w, s, b)
    assert empty.shape == (0, n)


def test_host_buffer_mlp_entry_point(cuda_device):
    """mt_affine_mlp_host: activations, residual and result in page-locked host memory, one call."""
    hidden, inter = 1024, 2048
    gate, up, down = synth.mlp_weights(310, hidden, inter, cuda_device)
    on_device = B.mlx_affine_mlp_executor(synth.activations(1, 1, hidden, cuda_device), *gate, *up, *down, None)
    from_host = B.mlx_affine_mlp_host_executor(8, hidden, *gate, *up, *down)
    for rows in (1, 3, 8):
        x = synth.activations(20 + rows, rows, hidden, cuda_device)
        res = synth.activations(30 + rows, rows, hidden, cuda_device)
        hx, hr = x.cpu().pin_memory(), res.cpu().pin_memory()
        out = torch.empty((rows, hidden), dtype=torch.bfloat16).pin_memory()
        from_host(hx, hr, out)
        torch.cuda.synchronize()
        assert_bit_equal(out.to(cuda_device), on_device(x, res), f"host entry point, rows={rows}")
        from_host(hx, None, out)
        torch.cuda.synchronize()
        assert_bit_equal(out.to(cuda_device), on_device(x, None), f"host entry point without residual, rows={rows}")
    # Activations and residual as two views of one page-locked buffer travel in one copy.
    both = torch.empty((2, rows, hidden), dtype=torch.bfloat16).pin_memory()
    both[0].copy_(x)
    both[1].copy_(res)
    from_host(both[0], both[1], out)
    torch.cuda.synchronize()
    assert_bit_equal(out.to(cuda_device), on_device(x, res), "host entry point, paired buffer")
    # Pageable host tensors are never handed to a kernel: they go through the copy engine.
    pageable_out = torch.empty((rows, hidden), dtype=torch.bfloat16)
    from_host(x.cpu(), res.cpu(), pageable_out)
    torch.cuda.synchronize()
    assert_bit_equal(pageable_out.to(cuda_device), on_device(x, res), "host entry point, pageable memory")
    with pytest.raises(ValueError):
        from_host(torch.empty((9, hidden), dtype=torch.bfloat16).pin_memory(), None,
                  torch.empty((9, hidden), dtype=torch.bfloat16).pin_memory())
    with pytest.raises(ValueError):
        from_host(x, None, out)  # device tensor
