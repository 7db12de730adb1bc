"""Shared helpers for the parity tests: torch tensors <-> the numpy oracle."""

import numpy as np
import torch

from metile_b200 import synth
from oracle import affine as oracle


def triple_np(triple):
    """(packed, scales, biases) torch tensors -> numpy (uint32, float32, float32)."""
    packed, scales, biases = triple
    return (
        packed.detach().cpu().numpy().astype(np.uint32),
        synth.to_numpy_f32(scales),
        synth.to_numpy_f32(biases),
    )


def f32(tensor):
    return synth.to_numpy_f32(tensor)


def assert_within(actual, reference, rel=2e-3, what=""):
    """Every |y - y_ref| <= rel * max|y_ref| + one bf16 ulp (see oracle.affine.within_tolerance)."""
    ok, ratio = oracle.within_tolerance(f32(actual) if isinstance(actual, torch.Tensor) else actual,
                                        reference, rel)
    assert ok, f"{what}: worst error is {ratio:.2f}x the allowed bound (rel={rel:g})"
    return ratio


def assert_bit_equal(a, b, what=""):
    a16 = a.detach().cpu().contiguous().view(torch.uint16)
    b16 = b.detach().cpu().contiguous().view(torch.uint16)
    mismatches = int((a16 != b16).sum())
    assert mismatches == 0, f"{what}: {mismatches} of {a16.numel()} outputs differ bitwise"
