"""GPU tests of the failure paths that must end in a status code, never in a fault or a hang:
the bounded device-side waits (made to run out by the library's own self-test kernels, whose waits
nothing can satisfy), the reset that follows, and the argument checks in front of every raw pointer."""

import ctypes

import pytest
import torch

from metile_b200 import _lib, backends as B, synth
from metile_b200.kernels import affine_qmv as k_qmv
from metile_b200.kernels import mlp as k_mlp
from oracle import affine as A
from tests.helpers import assert_bit_equal, assert_within, f32, triple_np

pytestmark = pytest.mark.gpu

WAIT_SELFTEST = 0x7E1
WAIT_GRID_BARRIER = 0x203


def _stream(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def test_a_wait_nothing_satisfies_gives_up_with_a_status(cuda_device):
    lib = _lib.load()
    ok, _ = _lib.device_status()
    assert ok
    assert lib.mt_selftest_bounded_wait(0, 2000, _stream(cuda_device)) == 0  # 2 ms limit
    words = (ctypes.c_uint * 4)()
    assert lib.mt_device_status(words, 0) == -8          # synchronises; the kernel returned by itself
    assert words[0] == WAIT_SELFTEST and words[1] == 0    # code and block of the waiter
    assert "wait gave up" in _lib.status_string(-8)
    assert lib.mt_device_status(words, 1) == -8          # still recorded; this call clears it
    ok, words = _lib.device_status()
    assert ok and words[0] == 0
    # The context is intact: an ordinary projection still runs and is right.
    weight = synth.affine_weight(3, 128, 256, cuda_device)
    x = synth.activations(4, 2, 256, cuda_device)
    assert_within(B.mlx_affine_qmv(x, *weight), A.qmm(f32(x), *triple_np(weight), weights="bf16"))
    assert lib.mt_selftest_bounded_wait(0, 0, None) == -1 and lib.mt_selftest_bounded_wait(7, 10, None) == -1


def test_grid_barrier_that_gives_up_is_repaired_by_the_reset(cuda_device):
    """A grid barrier whose wait runs out leaves its counter short.  The reset zeroes the counters,
    so every later single-launch MLP -- whichever of the 64 rotating counters it draws -- is right."""
    lib = _lib.load()
    hidden, inter = 1024, 2048
    gate, up, down = synth.mlp_weights(77, hidden, inter, cuda_device)
    x = synth.activations(5, 1, hidden, cuda_device)
    res = synth.activations(6, 1, hidden, cuda_device)
    execute = B.mlx_affine_mlp_executor(x, *gate, *up, *down, res)
    assert lib.mt_affine_mlp_launches(1, hidden, inter, 0) == 1
    before = execute(x, res)
    torch.cuda.synchronize()
    assert lib.mt_selftest_bounded_wait(1, 2000, _stream(cuda_device)) == 0
    words = (ctypes.c_uint * 4)()
    assert lib.mt_device_status(words, 1) == -8 and words[0] == WAIT_GRID_BARRIER
    for _ in range(70):  # more launches than counters
        assert_bit_equal(execute(x, res), before, "single-launch MLP after a barrier time-out and reset")
    ok, words = _lib.device_status()
    assert ok, [hex(w) for w in words]


def test_pointers_are_checked_before_any_launch(cuda_device):
    weight = synth.affine_weight(3, 128, 256, cuda_device)
    x = synth.activations(4, 2, 256, cuda_device)
    out = torch.empty((2, 128), dtype=torch.bfloat16, device=cuda_device)
    with pytest.raises(ValueError, match="CUDA device"):
        B.mlx_affine_residual_qmv(x, *weight, torch.zeros((2, 128), dtype=torch.bfloat16))  # host residual
    with pytest.raises(ValueError, match="CUDA device"):
        B.mlx_add_rms_norm(x, x, torch.ones(256, dtype=torch.bfloat16), 1e-6)                # host norm weight
    with pytest.raises(ValueError):
        k_qmv.affine_residual_qmv(x, *weight, torch.zeros(128, dtype=torch.bfloat16, device=cuda_device), out,
                                  256, 128)                                                    # short residual
    gate, up, down = synth.mlp_weights(9, 256, 512, cuda_device)
    hidden = torch.empty((2, 512), dtype=torch.bfloat16, device=cuda_device)
    y = torch.empty((2, 256), dtype=torch.bfloat16, device=cuda_device)
    with pytest.raises(ValueError):
        k_mlp.affine_swiglu_mlp(x, *gate, *up, *down, torch.zeros(256, dtype=torch.bfloat16, device=cuda_device),
                                hidden, y)                                                     # short residual
    with pytest.raises(ValueError):
        k_mlp.affine_swiglu_mlp(x, *gate, *up, *down, None, hidden, y.float())                # wrong output dtype
    execute = B.mlx_affine_mlp_executor(x, *gate, *up, *down, x)
    with pytest.raises(ValueError):
        execute(x.cpu(), None)                                                                 # host activations
    with pytest.raises(ValueError, match="CUDA device"):
        execute(x, x.cpu())                                                                    # host residual
    ok, words = _lib.device_status()
    assert ok, words


def test_null_or_misaligned_down_operands_are_refused_before_the_first_kernel(cuda_device):
    """mt_affine_mlp checks all three projections up front: a bad down operand must not leave the
    gate|up kernel queued and the workspace half written."""
    lib = _lib.load()
    hidden, inter, rows = 256, 512, 2
    gate, up, down = synth.mlp_weights(9, hidden, inter, cuda_device)
    x = synth.activations(4, rows, hidden, cuda_device)
    workspace = torch.full((rows, inter), 7.0, dtype=torch.bfloat16, device=cuda_device)
    out = torch.empty((rows, hidden), dtype=torch.bfloat16, device=cuda_device)
    p = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())  # noqa: E731
    for flags in (0, _lib.FLAG_FORCE_GEMV, _lib.FLAG_FORCE_UMMA):
        for bad in ("null", "misaligned"):
            down_w = None if bad == "null" else ctypes.c_void_p(down[0].data_ptr() + 4)
            code = lib.mt_affine_mlp(p(x), p(gate[0]), p(gate[1]), p(gate[2]), p(up[0]), p(up[1]), p(up[2]), down_w,
                                     p(down[1]), p(down[2]), None, p(workspace), workspace.numel() * 2, p(out), rows,
                                     hidden, inter, 64, 4, flags, _stream(cuda_device))
            assert code in (-6, -2), (flags, bad, code)
    torch.cuda.synchronize()
    assert bool((workspace == 7.0).all()), "a refused call must not have queued the gate|up kernel"


def test_a_call_on_a_device_that_is_not_current(cuda_device):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs a second GPU")
    other = torch.device("cuda", 1)
    weight = synth.affine_weight(3, 128, 256, other)
    x = synth.activations(4, 2, 256, other)
    assert torch.cuda.current_device() == 0
    y = B.mlx_affine_qmv(x, *weight)
    assert y.device == other
    assert_within(y, A.qmm(f32(x), *triple_np(weight), weights="bf16"))
    gate, up, down = synth.mlp_weights(9, 1024, 2048, other)
    x1 = synth.activations(5, 1, 1024, other)
    y1 = B.mlx_affine_mlp_executor(x1, *gate, *up, *down, x1)(x1, x1)
    assert_within(y1, A.mlp(f32(x1), triple_np(gate), triple_np(up), triple_np(down), f32(x1)), rel=4e-3)
    assert torch.cuda.current_device() == 0
