"""World-size-2 (and 4) gloo tests of the tensor-parallel sharding on CPU.

The CUDA operators are replaced by the numpy oracle through the constructor's injection points,
so what is tested here is the host logic: which rows / packed columns each rank owns, that the
residual enters exactly once, and that one all-reduce of the partial down outputs reproduces
the unsharded MLP.
"""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from metile_b200 import synth, tp
from oracle import affine as A
from tests.helpers import f32, triple_np

HIDDEN, INTER, ROWS = 128, 512, 3


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_swiglu(values, gw, gs, gb, uw, us, ub):
    out = A.swiglu_fused(f32(values), triple_np((gw, gs, gb)), triple_np((uw, us, ub)))
    return torch.from_numpy(out).to(torch.bfloat16)


def _oracle_down(hidden, w, s, b, residual):
    out = A.qmm(f32(hidden), *triple_np((w, s, b)), residual=None if residual is None else f32(residual),
                out="f32")
    return torch.from_numpy(out)  # fp32 partials keep the CPU check tight


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        gate, up, down = synth.mlp_weights(7, HIDDEN, INTER)
        x = synth.activations(1, ROWS, HIDDEN)
        res = synth.activations(2, ROWS, HIDDEN)
        module = tp.TensorParallelMLP.from_full(gate, up, down, "cpu", rank, world, swiglu_fn=_oracle_swiglu,
                                                down_fn=_oracle_down)
        assert module.gate[0].shape == (INTER // world, HIDDEN // 8)
        assert module.down[0].shape == (HIDDEN, INTER // world // 8)
        assert module.down[1].shape == (HIDDEN, INTER // world // 64)
        y = module(x, res)
        results[rank] = y.numpy().copy()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_mlp_matches_unsharded(world):
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    gate, up, down = synth.mlp_weights(7, HIDDEN, INTER)
    x, res = synth.activations(1, ROWS, HIDDEN), synth.activations(2, ROWS, HIDDEN)
    hidden = A.swiglu_fused(f32(x), triple_np(gate), triple_np(up))
    full = A.qmm(hidden, *triple_np(down), residual=f32(res), out="f32")
    for rank in range(world):
        np.testing.assert_allclose(results[rank], full, rtol=1e-5, atol=1e-5)


def test_shard_bounds_reject_cut_groups():
    assert tp.shard_bounds(27648, 3, 8) == (3 * 3456, 4 * 3456)
    with pytest.raises(ValueError):
        tp.shard_bounds(8960, 0, 8)  # 8960 / 8 = 1120 is not a multiple of 64
    gate = synth.affine_weight(1, 256, 128)
    down = synth.affine_weight(2, 128, 256)
    lo = tp.shard_gate_up(gate, 1, 2)
    assert lo[0].shape == (128, 16) and lo[0].is_contiguous()
    part = tp.shard_down(down, 1, 2)
    assert part[0].shape == (128, 16) and part[1].shape == (128, 2)
    assert (part[0] == down[0][:, 16:]).all()


def test_rank_failure_is_reported_on_the_host():
    """A rank that never joins: the others see a timeout from the process group on the host."""
    import datetime

    port = _free_port()

    def lonely(rank, world):
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        with pytest.raises(Exception):
            dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=2))

    lonely(0, 2)
