"""CPU tests of the argument checks that guard every raw pointer handed to the C ABI, and of the
device guard around each call.  No kernel runs here."""

import contextlib
import types

import pytest
import torch

from metile_b200 import backends
from metile_b200.backends import _common
from metile_b200.kernels import add_rmsnorm as k_add_rmsnorm
from metile_b200.kernels import affine_qmv as k_qmv
from metile_b200.kernels import mlp as k_mlp

CUDA0 = types.SimpleNamespace(device=torch.device("cuda", 0))


def test_pointer_check_rejects_host_foreign_short_and_mistyped_tensors():
    host = torch.zeros(8, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="CUDA device"):
        _common.require_on_device(host, CUDA0, "residual")
    with pytest.raises(TypeError):
        _common.require_on_device([1, 2, 3], CUDA0, "residual")
    _common.require_on_device(None, CUDA0, "residual")  # optional operands stay optional
    # A tensor that claims another GPU: checked on a stand-in, no second device is needed.
    other = types.SimpleNamespace(device=torch.device("cuda", 1), is_cuda=True)
    fake = torch.zeros(8, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="CUDA device"):
        _common.require_on_device(fake, other, "residual")
    # The remaining clauses, with the device clause satisfied by a stand-in.
    like = types.SimpleNamespace(device=fake.device)
    original = torch.Tensor.is_cuda
    try:
        torch.Tensor.is_cuda = property(lambda self: True)
        with pytest.raises(ValueError, match="needs at least"):
            _common.require_on_device(fake, like, "Out", min_numel=9)
        with pytest.raises(ValueError, match="must be torch.bfloat16"):
            _common.require_on_device(fake.float(), like, "Out", dtype=torch.bfloat16)
        with pytest.raises(ValueError, match="contiguous"):
            _common.require_on_device(torch.zeros((4, 4), dtype=torch.bfloat16).t(), like, "Out")
        _common.require_on_device(fake, like, "Out", dtype=torch.bfloat16, min_numel=8)
    finally:
        torch.Tensor.is_cuda = original


def test_operators_refuse_host_activations_before_any_launch():
    x = torch.zeros((1, 64), dtype=torch.bfloat16)
    w = torch.zeros((64, 8), dtype=torch.int32)
    s = torch.zeros((64, 1), dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="CUDA"):
        backends.mlx_affine_qmv(x, w, s, s)
    with pytest.raises(ValueError, match="CUDA"):
        backends.mlx_add_rms_norm(x, x, torch.ones(64, dtype=torch.bfloat16), 1e-6)
    with pytest.raises(ValueError, match="CUDA"):
        k_qmv.affine_qmv(x, w, s, s, torch.zeros((1, 64), dtype=torch.bfloat16), 64, 64)
    with pytest.raises(ValueError, match="CUDA"):
        k_add_rmsnorm.add_rmsnorm(x, x, torch.ones(64, dtype=torch.bfloat16), x.clone(), x.clone(), 64, 1e-6)
    with pytest.raises(ValueError, match="CUDA"):
        k_mlp.matmul_silu(x, torch.zeros((64, 8), dtype=torch.bfloat16), torch.zeros((1, 8), dtype=torch.bfloat16),
                          1, 8, 64)


def test_every_call_runs_with_the_tensors_device_current(monkeypatch):
    """`launch` makes the tensors' device current around the C call and passes that device's stream."""
    events = []

    @contextlib.contextmanager
    def fake_device(device):
        events.append(("enter", device))
        yield
        events.append(("exit", device))

    monkeypatch.setattr(torch.cuda, "device", fake_device)
    monkeypatch.setattr(torch.cuda, "current_device", lambda: 0)
    monkeypatch.setattr(_common, "stream_pointer", lambda device: ("stream-of", device))

    def entry_point(*arguments):
        events.append(("call", arguments))
        return 0

    device = torch.device("cuda", 1)
    assert _common.launch(entry_point, device, 1, 2, 3) == 0
    assert events == [("enter", device), ("call", (1, 2, 3, ("stream-of", device))), ("exit", device)]
    # Already current: no switch, same stream argument.
    events.clear()
    here = torch.device("cuda", 0)
    assert _common.launch(entry_point, here, 4) == 0
    assert events == [("call", (4, ("stream-of", here)))]
