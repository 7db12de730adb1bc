"""GPU parity of the named workloads at their full shapes against the CPU oracle -- every piece of
the Qwen2.5-1.5B-shaped decoder block (q/o 1536x1536, k/v 1536->256, MLP 1536/8960, add+RMSNorm at 512
and 16 rows, and the MLP half of the block end to end), and the Qwen2.5-32B-shaped MLP (5120 / 27648)
unsharded and at the shard shapes of a tensor-parallel run -- plus the table of measured error
ratios and the count of cross-regime bit mismatches.

Checker: the C + OpenMP port under oracle/ (fp32 accumulate, exact weights) for the large shapes, the
numpy oracle (float64) where a bf16-rounded-weight variant is needed."""

import json
import os

import numpy as np
import pytest
import torch

from metile_b200 import _lib, backends as B, synth
from oracle import affine as A
from oracle import cport
from tests.helpers import assert_bit_equal, assert_within, f32, triple_np

pytestmark = pytest.mark.gpu
RATIOS = {}


def bits(triple):
    return triple[0].cpu().numpy(), synth.to_numpy_bits(triple[1]), synth.to_numpy_bits(triple[2])


def record(name, ratio, rel):
    """Worst |error| / bound of a check, kept for the table written at the end of the module."""
    RATIOS[name] = {"worst_over_bound": round(float(ratio), 4), "rel": rel}


@pytest.fixture(scope="module", autouse=True)
def write_ratio_table():
    yield
    out = os.environ.get("METILE_REPORT_DIR", "")
    if RATIOS and os.path.isdir(out):
        with open(os.path.join(out, "parity_ratios.json"), "w") as handle:
            json.dump(RATIOS, handle, indent=1, sort_keys=True)


@pytest.mark.parametrize("name,k,n", [("q_proj", 1536, 1536), ("k_proj", 1536, 256), ("o_proj", 1536, 1536)])
@pytest.mark.parametrize("rows", [16, 512])
def test_qwen_block_projections(cuda_device, name, k, n, rows):
    weight = synth.affine_weight({"q_proj": 1, "k_proj": 2, "o_proj": 4}[name], n, k, cuda_device)
    x = synth.activations(70, rows, k, cuda_device, std=0.5)
    y = B.mlx_affine_qmv(x, *weight)
    reference = A.bf16_from_bits(cport.qmm(synth.to_numpy_bits(x), *bits(weight)))
    record(f"block {name} {rows} rows vs C port", assert_within(y, reference, what=f"{name} {rows}x{k}x{n}"), 2e-3)
    assert A.accuracy_compatible(f32(y), reference)


@pytest.mark.parametrize("rows", [16, 512])
def test_qwen_block_mlp_half_end_to_end(cuda_device, rows):
    """h = x + attn;  out = h + down(swiglu(rmsnorm(h))): the fused add+RMSNorm feeding the fused MLP
    with the residual in the down projection's epilogue, against the oracle's composition."""
    hidden, inter, eps = 1536, 8960, 1e-6
    gate, up, down = synth.mlp_weights(5, hidden, inter, cuda_device)
    norm_w = synth.norm_weight(9, hidden, cuda_device)
    x = synth.activations(71, rows, hidden, cuda_device, std=0.5)
    attn = synth.activations(72, rows, hidden, cuda_device, std=0.5)
    summed, normed = B.mlx_add_rms_norm(x, attn, norm_w, eps)
    out = B.mlx_affine_mlp_executor(normed, *gate, *up, *down, summed)(normed, summed)
    o_sum, o_norm = A.add_rmsnorm(f32(x), f32(attn), f32(norm_w), eps)
    assert (f32(summed) == o_sum).all(), "Sum is the exact bf16 add"
    record(f"block add_rmsnorm {rows} rows", assert_within(normed, o_norm, what="add_rmsnorm"), 2e-3)
    # The MLP on the kernel's own normalised rows (so that only the MLP's arithmetic is compared).
    reference = A.bf16_from_bits(cport.mlp(synth.to_numpy_bits(normed), *[bits(t) for t in (gate, up, down)],
                                           synth.to_numpy_bits(summed)))
    record(f"block MLP 1536/8960 {rows} rows vs C port",
           assert_within(out, reference, rel=3e-3, what=f"block MLP {rows} rows"), 3e-3)
    assert A.affine_swiglu_compatible(f32(out), reference)


@pytest.mark.parametrize("rows", [1, 16, 128])
def test_qwen32b_mlp_unsharded(cuda_device, rows):
    """hidden 5120 / intermediate 27648 on one GPU, through mt_affine_mlp."""
    hidden, inter = 5120, 27648
    gate, up, down = synth.mlp_weights(100, hidden, inter, cuda_device)
    x = synth.activations(5, rows, hidden, cuda_device)
    res = synth.activations(6, rows, hidden, cuda_device)
    y = B.mlx_affine_mlp_executor(x, *gate, *up, *down, res)(x, res)
    reference = A.bf16_from_bits(cport.mlp(synth.to_numpy_bits(x), *[bits(t) for t in (gate, up, down)],
                                           synth.to_numpy_bits(res)))
    record(f"MLP 5120/27648 {rows} rows vs C port", assert_within(y, reference, rel=3e-3, what=f"32B MLP M={rows}"), 3e-3)
    assert A.affine_swiglu_compatible(f32(y), reference)


@pytest.mark.parametrize("world", [2, 8])
def test_qwen32b_mlp_shard_shapes_sum_to_the_unsharded_result(cuda_device, world):
    """The tensor-parallel partition on ONE GPU: every rank's shard (gate|up column slice, down row
    slice) runs through the same kernels, the partial outputs are added in rank order in fp32, and the
    sum is compared with the unsharded oracle.  The shard shapes are 5120 / 13824 and 5120 / 3456."""
    from metile_b200 import tp as tensor_parallel

    hidden, inter, rows = 5120, 27648, 16
    gate, up, down = synth.mlp_weights(100, hidden, inter, cuda_device)
    x = synth.activations(5, rows, hidden, cuda_device)
    res = synth.activations(6, rows, hidden, cuda_device)
    total = torch.zeros((rows, hidden), dtype=torch.float32, device=cuda_device)
    for rank in range(world):
        g, u, d = tensor_parallel.shard_mlp_weights(gate, up, down, rank, world)
        assert g[0].shape[0] == inter // world and d[0].shape[1] == inter // world // 8
        execute = B.mlx_affine_mlp_executor(x, *g, *u, *d, res)
        total += execute(x, res if rank == 0 else None).float()
    reference = A.bf16_from_bits(cport.mlp(synth.to_numpy_bits(x), *[bits(t) for t in (gate, up, down)],
                                           synth.to_numpy_bits(res)))
    record(f"MLP 5120/27648 as {world} shards, fp32 sum vs C port",
           assert_within(total.to(torch.bfloat16), reference, rel=3e-3, what=f"tp{world} shards"), 3e-3)


def test_cross_regime_bit_mismatches_are_counted(cuda_device):
    """The default dispatch serves one row, two to eight rows and more rows from different kernels
    (CUDA-core FMA, mma.sync, tcgen05), whose fp32 orders differ: a row's bits may differ between
    regimes (always within tolerance).  Count how many outputs do, and check that the invariant mode
    (one kernel family for every batch size) has none."""
    hidden, inter = 2048, 8192
    gate, up, down = synth.mlp_weights(100, hidden, inter, cuda_device)
    x = synth.activations(5, 128, hidden, cuda_device)
    res = synth.activations(6, 128, hidden, cuda_device)
    execute = B.mlx_affine_mlp_executor(x[:1], *gate, *up, *down, res[:1])
    alone = execute(x[:1], res[:1])
    counts = {}
    for rows in (2, 8, 16, 128):
        batch = execute(x[:rows], res[:rows])
        counts[rows] = int((batch[:1].view(torch.uint16) != alone.view(torch.uint16)).sum())
        assert_within(batch[:1], f32(alone), rel=3e-3, what=f"row 0 alone vs in a batch of {rows}")
    RATIOS["cross-regime mismatches of row 0 (of 2048 outputs), default dispatch"] = counts
    with B.batch_invariant():
        alone_inv = execute(x[:1], res[:1])
        for rows in (2, 8, 16, 128):
            assert_bit_equal(execute(x[:rows], res[:rows])[:1], alone_inv, f"invariant mode, batch of {rows}")
