"""Tensor-parallel INT4 SwiGLU MLP across the GPUs of one node (one process per GPU).

The reference is single-device; this is the multi-GPU form of its fused MLP
(metile/backends/mlx_quantized.py:1770, mlx_affine_mlp_executor) for shapes too large for one
GPU's bandwidth budget:

  * gate and up are COLUMN-sharded: rank r of t owns intermediate rows [r*I/t, (r+1)*I/t) of both,
    so SwiGLU -- elementwise over the intermediate axis -- stays local;
  * down is ROW-sharded: rank r owns the matching K slice [r*I/t, (r+1)*I/t) of every output row,
    i.e. packed columns [r*I/(8t), ...) and scale/bias columns [r*I/(64t), ...); I/t must be a
    multiple of 64 so a slice never cuts a quantisation group;
  * each rank's down output is a partial sum over its K slice; ONE all-reduce (NCCL over
    NVLink/NVSwitch) per MLP adds them.  The residual enters on rank 0 only, through the down
    kernel's fused residual epilogue, so no extra elementwise kernel runs after the reduce.

Partials are bf16 (the reduce runs in bf16).  The order in which NCCL sums ranks may change
with message size, so bit-exact batch invariance is a single-GPU property; across TP ranks
results agree with the single-GPU MLP to the 2e-3-of-peak tolerance.
"""

from __future__ import annotations

import torch

_cpu_cache = {}


def shard_bounds(intermediate, rank, world, group_size=64):
    if intermediate % (world * group_size):
        raise ValueError(
            f"intermediate size {intermediate} cannot be split into {world} shards of whole "
            f"{group_size}-wide quantisation groups"
        )
    width = intermediate // world
    return rank * width, (rank + 1) * width


def shard_gate_up(triple, rank, world, group_size=64):
    """Rows [lo, hi) of a [I, H/8] packed weight and its [I, H/64] scales / biases."""
    packed, scales, biases = triple
    lo, hi = shard_bounds(packed.shape[0], rank, world, group_size)
    return packed[lo:hi].contiguous(), scales[lo:hi].contiguous(), biases[lo:hi].contiguous()


def shard_down(triple, rank, world, group_size=64):
    """K slice [lo, hi) of a [H, I/8] packed weight: packed columns lo/8.., parameter columns lo/64.."""
    packed, scales, biases = triple
    intermediate = packed.shape[1] * 8
    lo, hi = shard_bounds(intermediate, rank, world, group_size)
    return (packed[:, lo // 8:hi // 8].contiguous(), scales[:, lo // group_size:hi // group_size].contiguous(),
            biases[:, lo // group_size:hi // group_size].contiguous())


def shard_mlp_weights(gate, up, down, rank, world, group_size=64):
    """This rank's (gate, up, down) shards of full weight triples."""
    return (shard_gate_up(gate, rank, world, group_size), shard_gate_up(up, rank, world, group_size),
            shard_down(down, rank, world, group_size))


class TensorParallelMLP:
    """down(swiglu(x)) + residual with the weights sharded over `world` ranks."""

    def __init__(self, gate, up, down, rank, world, *, group=None, swiglu_fn=None, down_fn=None,
                 all_reduce_fn=None):
        """`swiglu_fn(values, gate..., up...)`, `down_fn(hidden, w, s, b, residual_or_None)` and
        `all_reduce_fn(tensor)` default to the CUDA operators and torch.distributed; they can be
        replaced to exercise the sharding logic without a GPU."""
        self.gate, self.up, self.down = gate, up, down
        self.rank, self.world, self.group = rank, world, group
        # With the CUDA operators, the shard's MLP is ONE C-ABI call on a bound executor (both kernels,
        # workspace owned by the executor, the residual in rank 0's down epilogue): one Python dispatch
        # and one all-reduce per MLP.  Injected stand-ins take the two-step path.
        self._executor = None
        self._swiglu, self._down = swiglu_fn, down_fn
        self._all_reduce = all_reduce_fn or self._dist_all_reduce

    def _bound_executor(self, values):
        if self._executor is None:
            from .backends.cuda_quantized import mlx_affine_mlp_executor

            self._executor = mlx_affine_mlp_executor(values, *self.gate, *self.up, *self.down, None)
        return self._executor

    def _dist_all_reduce(self, tensor):
        if self.world > 1:
            import torch.distributed as dist

            dist.all_reduce(tensor, op=dist.ReduceOp.SUM, group=self.group)
        return tensor

    @classmethod
    def from_full(cls, gate, up, down, device, rank, world, **kwargs):
        """Cut this rank's shards out of full (unsharded) weight triples and move them to `device`."""
        move = lambda triple: tuple(t.to(device) for t in triple)  # noqa: E731
        return cls(move(shard_gate_up(gate, rank, world)), move(shard_gate_up(up, rank, world)),
                   move(shard_down(down, rank, world)), rank, world, **kwargs)

    @classmethod
    def from_seed(cls, seed, hidden, intermediate, device, rank, world, **kwargs):
        """Seeded synthetic weights; every rank slices the SAME full tensors, so results are
        comparable across TP degrees."""
        from . import synth

        key = (seed, hidden, intermediate, rank, world)
        if key not in _cpu_cache:
            gate, up, down = synth.mlp_weights(seed, hidden, intermediate)
            _cpu_cache.clear()
            _cpu_cache[key] = (shard_gate_up(gate, rank, world), shard_gate_up(up, rank, world),
                               shard_down(down, rank, world))
        gate, up, down = _cpu_cache[key]
        move = lambda triple: tuple(t.to(device) for t in triple)  # noqa: E731
        return cls(move(gate), move(up), move(down), rank, world, **kwargs)

    def partial(self, values, residual=None):
        """This rank's partial output [M, H] (bf16): its K slice of the down projection, plus the
        residual on rank 0."""
        mine = residual if self.rank == 0 else None
        if self._swiglu is None and self._down is None:
            return self._bound_executor(values)(values, mine)
        hidden = self._swiglu(values, *self.gate, *self.up)
        return self._down(hidden, *self.down, mine)

    def __call__(self, values, residual=None):
        return self._all_reduce(self.partial(values, residual))
