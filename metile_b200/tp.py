"""Tensor-parallel INT4 SwiGLU MLP across the GPUs of one node (one process per GPU).

The reference is single-device; this is the multi-GPU form of its fused MLP
(metile/backends/mlx_quantized.py:1770, mlx_affine_mlp_executor) for shapes too large for one
GPU's bandwidth budget:

  * gate and up are COLUMN-sharded: rank r of t owns intermediate rows [r*I/t, (r+1)*I/t) of both,
    so SwiGLU -- elementwise over the intermediate axis -- stays local;
  * down is ROW-sharded: rank r owns the matching K slice [r*I/t, (r+1)*I/t) of every output row,
    i.e. packed columns [r*I/(8t), ...) and scale/bias columns [r*I/(64t), ...); I/t must be a
    multiple of 64 so a slice never cuts a quantisation group;
  * each rank's down output is a partial sum over its K slice; ONE sum over the ranks per MLP adds
    them.  The residual enters on rank 0 only, through the down kernel's fused residual epilogue, so
    no extra elementwise kernel runs after the sum.

The sum is the library's own one-shot exchange (`PeerAllReduce`, mt_peer_all_reduce): one kernel per
rank stores the bf16 partial into every peer's memory over NVLink, waits for the peers' stores and
adds the partials in RANK ORDER in fp32.  Every rank gets the same bits and the order does not change
with the message size, so a row's result does not depend on the batch it arrives in as long as the
shard kernels are batch-invariant themselves (`batch_invariant()`).  `all_reduce="nccl"` selects
torch.distributed's all-reduce instead, whose summation order is NCCL's choice.  Either way the
partials are rounded to bf16 before they are added, so the sharded result agrees with the single-GPU
MLP to the tolerance of two bf16 roundings more, not bit for bit.
"""

from __future__ import annotations

import ctypes

import torch

_cpu_cache = {}


class PeerAllReduce:
    """In-place sum of a bf16 tensor over the ranks of `group` through peer memory (mt_peer_all_reduce).

    Construction is collective: every rank allocates its receive buffer in the library, and the CUDA
    IPC handles are exchanged with `all_gather_object`.  `max_elements` bounds the message; larger
    tensors are refused by the library (-7).  Every rank must make the same calls in the same order,
    on one stream (calls of one group must not overlap on a GPU); a CUDA graph containing calls may be
    replayed, the same number of times on every rank."""

    MODES = {"auto": 0, "one_shot": 1, "two_shot": 2}

    def __init__(self, device, rank, world, max_elements, *, group=None, limit_ms=1000, mode="auto"):
        import torch.distributed as dist

        from . import _lib
        from .backends import _common

        self._lib, self._common = _lib.load(), _common
        self.device, self.rank, self.world, self.group = torch.device(device), rank, world, group
        self.max_elements, self.limit_ms = int(max_elements), int(limit_ms)
        slot_bytes = (self.max_elements * 2 + 15) // 16 * 16
        self._handle = ctypes.c_void_p()
        mine = ctypes.create_string_buffer(64)
        with torch.cuda.device(self.device):
            _lib.check(self._lib.mt_peer_group_create(rank, world, slot_bytes, ctypes.byref(self._handle), mine),
                       "mt_peer_group_create")
        gathered = [None] * world
        if world > 1:
            dist.all_gather_object(gathered, mine.raw, group=group)
        else:
            gathered[0] = mine.raw
        with torch.cuda.device(self.device):
            _lib.check(self._lib.mt_peer_group_connect(self._handle, b"".join(gathered)), "mt_peer_group_connect")
        if mode not in self.MODES:
            raise ValueError('mode must be "auto", "one_shot" or "two_shot"')
        _lib.check(self._lib.mt_peer_group_set_mode(self._handle, self.MODES[mode]), "mt_peer_group_set_mode")

    def __call__(self, tensor):
        if tensor.dtype != torch.bfloat16 or not tensor.is_cuda or tensor.device != self.device:
            raise ValueError(f"PeerAllReduce expects a bfloat16 tensor on {self.device}")
        if not tensor.is_contiguous():
            raise ValueError("PeerAllReduce expects a contiguous tensor")
        from . import _lib

        pointer = ctypes.c_void_p(tensor.data_ptr())
        _lib.check(self._common.launch(self._lib.mt_peer_all_reduce, self.device, self._handle, pointer, pointer,
                                       tensor.numel(), self.limit_ms), "mt_peer_all_reduce")
        return tensor

    def close(self):
        """Collective: waits for every rank, then releases the mappings and the buffer."""
        if self._handle:
            import torch.distributed as dist

            torch.cuda.synchronize(self.device)
            if self.world > 1:
                dist.barrier(group=self.group)
            with torch.cuda.device(self.device):
                self._lib.mt_peer_group_destroy(self._handle)
            self._handle = ctypes.c_void_p()


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


_peer_groups = {}


def shared_peer_all_reduce(device, rank, world, max_elements, group=None):
    """One PeerAllReduce per (device, process group, capacity), shared by every MLP of a model: the
    MLPs of consecutive layers run one after the other on one stream, so one buffer serves them all."""
    key = (str(device), rank, world, id(group), int(max_elements))
    if key not in _peer_groups:
        _peer_groups[key] = PeerAllReduce(device, rank, world, max_elements, group=group)
    return _peer_groups[key]


def close_peer_groups():
    """Collective: release every shared exchange buffer (call before destroying the process group)."""
    for key in sorted(_peer_groups):
        _peer_groups.pop(key).close()


class TensorParallelMLP:
    """down(swiglu(x)) + residual with the weights sharded over `world` ranks."""

    def __init__(self, gate, up, down, rank, world, *, group=None, swiglu_fn=None, down_fn=None,
                 all_reduce_fn=None, all_reduce="peer", max_rows=128):
        """`swiglu_fn(values, gate..., up...)`, `down_fn(hidden, w, s, b, residual_or_None)` and
        `all_reduce_fn(tensor)` default to the CUDA operators; they can be replaced to exercise the
        sharding logic without a GPU.  `all_reduce`: "peer" (the library's exchange through peer
        memory, for up to `max_rows` rows; more rows go through NCCL) or "nccl"."""
        if all_reduce not in ("peer", "nccl"):
            raise ValueError('all_reduce must be "peer" or "nccl"')
        self.gate, self.up, self.down = gate, up, down
        self.rank, self.world, self.group = rank, world, group
        # With the CUDA operators, the shard's MLP is ONE C-ABI call on a bound executor (both kernels,
        # workspace owned by the executor, the residual in rank 0's down epilogue): one Python dispatch
        # and one all-reduce per MLP.  Injected stand-ins take the two-step path.
        self._executor = None
        self._swiglu, self._down = swiglu_fn, down_fn
        self._all_reduce = all_reduce_fn or (self._peer_all_reduce if all_reduce == "peer" else self._dist_all_reduce)
        self._peer, self._max_rows = None, int(max_rows)

    def _bound_executor(self, values):
        if self._executor is None:
            from .backends.cuda_quantized import mlx_affine_mlp_executor

            self._executor = mlx_affine_mlp_executor(values, *self.gate, *self.up, *self.down, None)
        return self._executor

    def _peer_all_reduce(self, tensor):
        if self.world == 1:
            return tensor
        rows, hidden = tensor.numel() // tensor.shape[-1], tensor.shape[-1]
        if not tensor.is_cuda or rows > self._max_rows or hidden % 8:
            return self._dist_all_reduce(tensor)
        if self._peer is None:  # collective on first use: every rank reaches its first call together
            self._peer = shared_peer_all_reduce(tensor.device, self.rank, self.world, self._max_rows * hidden,
                                                self.group)
        return self._peer(tensor)

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
