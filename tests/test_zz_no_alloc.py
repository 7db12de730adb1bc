"""GPU test of mt_affine_mlp_static, the fused MLP for callers that may not allocate device
memory (allocation-free serving loops, plugins confined to a fixed arena).  The entry point keeps the hidden activations in an array compiled into the library.

Called through the C ABI with raw pointers, twice in a row with different shapes, and compared
with mt_affine_mlp (caller-owned workspace) on the same inputs: the two must agree bit for bit,
which is inside the 2e-3-of-peak bound the other parity tests use.  This file sorts last so that a
run stopping at the first failure has already run every other test.
"""

import ctypes

import pytest
import torch

from metile_b200 import _lib, synth
from oracle import affine as A
from tests.helpers import assert_bit_equal, assert_within, f32, triple_np

pytestmark = pytest.mark.gpu


def _p(tensor):
    return None if tensor is None else ctypes.c_void_p(tensor.data_ptr())


def _run_pair(lib, device, rows, hidden, inter, seed):
    gate, up, down = synth.mlp_weights(seed, hidden, inter, device)
    x = synth.activations(seed + 10, rows, hidden, device)
    res = synth.activations(seed + 11, rows, hidden, device)
    weights = [t for triple in (gate, up, down) for t in triple]
    stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)

    reference = torch.empty((rows, hidden), dtype=torch.bfloat16, device=device)
    workspace = torch.empty((rows, inter), dtype=torch.bfloat16, device=device)
    code = lib.mt_affine_mlp(_p(x), *[_p(t) for t in weights], _p(res), _p(workspace), workspace.numel() * 2,
                             _p(reference), rows, hidden, inter, 64, 4, 0, stream)
    assert code == 0, _lib.status_string(code)

    out = torch.full((rows, hidden), float("nan"), dtype=torch.bfloat16, device=device)
    code = lib.mt_affine_mlp_static(_p(x), *[_p(t) for t in weights], _p(res), _p(out), rows, hidden, inter, 64, 4,
                                    0, stream)
    assert code == 0, _lib.status_string(code)
    torch.cuda.synchronize()
    assert_bit_equal(out, reference, f"static vs workspace MLP, rows={rows}")
    oracle = A.mlp(f32(x), triple_np(gate), triple_np(up), triple_np(down), f32(res),
                   weights="exact" if rows <= 8 and lib.mt_affine_mlp_launches(rows, hidden, inter, 0) == 1 else "bf16")
    assert_within(out, oracle, rel=3e-3, what=f"static MLP vs oracle, rows={rows}")


def test_static_scratch_mlp_matches_workspace_mlp_twice(cuda_device):
    lib = _lib.load()
    limit = lib.mt_affine_mlp_static_max_bytes()
    assert limit == 4 << 20
    # Two calls in a row share the array: a larger problem first, then a smaller one whose hidden
    # activations overlap what the first call left behind.
    _run_pair(lib, cuda_device, rows=16, hidden=512, inter=2048, seed=300)   # two tcgen05 kernels
    _run_pair(lib, cuda_device, rows=1, hidden=2048, inter=8192, seed=400)   # one launch on CUDA cores
    _run_pair(lib, cuda_device, rows=4, hidden=1024, inter=2048, seed=500)   # one launch on mma.sync
    ok, words = _lib.device_status()
    assert ok, words


def test_static_scratch_rejects_oversized_problems(cuda_device):
    lib = _lib.load()
    one = ctypes.c_void_p(256)
    too_many_rows = (4 << 20) // (8192 * 2) + 1
    code = lib.mt_affine_mlp_static(*([one] * 12), too_many_rows, 2048, 8192, 64, 4, 0, None)
    assert code == -7 and "workspace" in _lib.status_string(code)
    assert lib.mt_affine_mlp_static(*([one] * 12), 0, 2048, 8192, 64, 4, 0, None) == 0
