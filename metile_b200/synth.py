"""Seeded synthetic tensors in the MLX affine INT4 layout, at the shapes the benchmarks name.

Data is generated on the CPU from `torch.Generator().manual_seed(seed)` so it is identical for
any GPU count, then moved to the requested device.
"""

from __future__ import annotations

import numpy as np
import torch

GROUP_SIZE = 64


def pack_nibbles(quantized):
    """int tensor [N, K] with values 0..15 -> torch.uint32 [N, K/8], nibble e of word j = k 8j+e."""
    q = quantized.to(torch.int64).reshape(quantized.shape[0], -1, 8).numpy().astype(np.uint32)
    shifts = np.arange(0, 32, 4, dtype=np.uint32)
    return torch.from_numpy(np.bitwise_or.reduce(q << shifts, axis=-1).astype(np.uint32))


def affine_weight(seed, n, k, device="cpu"):
    """(packed u32 [N,K/8], scales bf16 [N,K/64], biases bf16 [N,K/64]).

    q uniform 0..15; scale ~ U(0.002, 0.02); bias = -8*scale + N(0, 1e-3)."""
    gen = torch.Generator().manual_seed(int(seed))
    q = torch.randint(0, 16, (n, k), generator=gen, dtype=torch.int64)
    scales = (torch.rand((n, k // GROUP_SIZE), generator=gen) * 0.018 + 0.002).to(torch.bfloat16)
    noise = torch.randn((n, k // GROUP_SIZE), generator=gen) * 1e-3
    biases = (-8.0 * scales.float() + noise).to(torch.bfloat16)
    return pack_nibbles(q).to(device), scales.to(device), biases.to(device)


def activations(seed, rows, width, device="cpu", std=1.0):
    gen = torch.Generator().manual_seed(int(seed))
    return (torch.randn((rows, width), generator=gen) * std).to(torch.bfloat16).to(device)


def norm_weight(seed, width, device="cpu"):
    gen = torch.Generator().manual_seed(int(seed))
    return (1.0 + 0.02 * torch.randn((width,), generator=gen)).to(torch.bfloat16).to(device)


def dense_weight(seed, n, k, device="cpu", std=0.02):
    gen = torch.Generator().manual_seed(int(seed))
    return (torch.randn((n, k), generator=gen) * std).to(torch.bfloat16).to(device)


def mlp_weights(seed, hidden, intermediate, device="cpu"):
    """gate/up [I, H] and down [H, I] affine triples, seeds seed, seed+1, seed+2."""
    return (
        affine_weight(seed, intermediate, hidden, device),
        affine_weight(seed + 1, intermediate, hidden, device),
        affine_weight(seed + 2, hidden, intermediate, device),
    )


def to_numpy_bits(tensor):
    """bf16 tensor -> numpy uint16 bit patterns (CPU copy)."""
    return tensor.detach().cpu().contiguous().view(torch.uint16).numpy()


def to_numpy_f32(tensor):
    """bf16 tensor -> numpy float32 (CPU copy)."""
    return tensor.detach().cpu().float().numpy()
