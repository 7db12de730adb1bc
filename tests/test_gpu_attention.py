"""GPU parity of decode attention, rotary embedding + KV append, and the fused decode step of an
attention module, against the numpy oracle (oracle/attention.py) on seeded inputs.

Tolerance: 2e-3 of the output peak plus one bf16 ulp (oracle.affine.within_tolerance), the bound the
projection tests use; attention outputs are convex combinations of bf16 values, so the peak is the
natural scale."""

import numpy as np
import pytest
import torch

from metile_b200 import _lib, backends as B, synth
from metile_b200.integrations import blocks, torch_lm
from oracle import affine as A
from oracle import attention as OA
from tests.helpers import assert_bit_equal, assert_within, f32

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def no_device_wait_gave_up(cuda_device):
    yield
    ok, words = _lib.device_status()
    assert ok, [hex(w) for w in words]


def qkv(seed, batch, q_heads, kv_heads, tokens, dim, device, capacity=None):
    capacity = capacity or tokens
    q = synth.activations(seed, batch * q_heads, dim, device).reshape(batch, q_heads, 1, dim)
    k = synth.activations(seed + 1, batch * kv_heads * capacity, dim, device).reshape(batch, kv_heads, capacity, dim)
    v = synth.activations(seed + 2, batch * kv_heads * capacity, dim, device).reshape(batch, kv_heads, capacity, dim)
    return q, k, v


@pytest.mark.parametrize("batch,q_heads,kv_heads,tokens,dim", [
    (2, 4, 2, 37, 64), (1, 8, 8, 130, 128), (3, 8, 1, 128, 64), (2, 12, 2, 257, 128), (1, 6, 2, 1, 128),
    (16, 12, 2, 2048, 128),  # the decode step of the Qwen2.5-1.5B-shaped block: 16 sequences at KV length 2048
])
def test_decode_attention_against_oracle(cuda_device, batch, q_heads, kv_heads, tokens, dim):
    q, k, v = qkv(11, batch, q_heads, kv_heads, tokens, dim, cuda_device)
    scale = dim ** -0.5
    out = B.mlx_attention_decode(q, k, v, scale=scale)
    assert out.shape == q.shape and out.dtype == torch.bfloat16
    assert_within(out, OA.attention_decode(f32(q), f32(k), f32(v), scale), what=f"decode attention {tokens} tokens")
    # The reference's admission rule and error behaviour.
    assert B.supports_attention_decode(q, k, v) is None
    assert B.supports_attention_decode(q, k, v, mask="causal") is not None
    with pytest.raises(ValueError):
        B.mlx_attention_decode(q.expand(-1, -1, 2, -1), k, v, scale=scale)  # two query rows


def test_decode_attention_on_an_in_place_cache_with_ragged_lengths(cuda_device):
    batch, q_heads, kv_heads, capacity, dim = 4, 12, 2, 600, 128
    q, k, v = qkv(21, batch, q_heads, kv_heads, 600, dim, cuda_device, capacity=capacity)
    scale = dim ** -0.5
    # A uniform prefix of a larger cache: the view is used in place (no copy), capacity read off its strides.
    used = 333
    out = B.mlx_attention_decode(q, k[:, :, :used], v[:, :, :used], scale=scale)
    assert_within(out, OA.attention_decode(f32(q), f32(k[:, :, :used]), f32(v[:, :, :used]), scale))
    # Ragged lengths, one per sequence.
    lengths = torch.tensor([1, 128, 129, 600], dtype=torch.int32, device=cuda_device)
    ragged = B.mlx_attention_decode(q, k, v, scale=scale, lengths=lengths)
    assert_within(ragged, OA.attention_decode(f32(q), f32(k), f32(v), scale, lengths=lengths.cpu().numpy()))
    # A sequence's bits depend on its own cache only: alone == inside the batch.
    for b in range(batch):
        alone = B.mlx_attention_decode(q[b:b + 1], k[b:b + 1], v[b:b + 1], scale=scale, lengths=lengths[b:b + 1])
        assert_bit_equal(alone, ragged[b:b + 1], f"sequence {b} alone vs in a batch of {batch}")


def test_rope_and_cache_append_against_oracle(cuda_device):
    batch, q_heads, kv_heads, capacity, dim, theta = 3, 12, 2, 64, 128, 1e6
    q = synth.activations(31, batch * q_heads, dim, cuda_device).reshape(batch, q_heads, dim)
    k = synth.activations(32, batch * kv_heads, dim, cuda_device).reshape(batch, kv_heads, dim)
    v = synth.activations(33, batch * kv_heads, dim, cuda_device).reshape(batch, kv_heads, dim)
    k_cache = synth.activations(34, batch * kv_heads * capacity, dim, cuda_device).reshape(batch, kv_heads, capacity, dim)
    v_cache = synth.activations(35, batch * kv_heads * capacity, dim, cuda_device).reshape(batch, kv_heads, capacity, dim)
    positions = torch.tensor([0, 17, 63], dtype=torch.int32, device=cuda_device)
    expect_k, expect_v = f32(k_cache).copy(), f32(v_cache).copy()
    rotated = B.rope_kv_append(q, k, v, positions, k_cache, v_cache, theta=theta)
    where = positions.cpu().numpy()
    assert_within(rotated, OA.rope(f32(q), where, theta), what="rotated query")
    OA.kv_append(expect_k, expect_v, OA.rope(f32(k), where, theta), f32(v), where)
    for b, position in enumerate(where.tolist()):
        assert_within(k_cache[b, :, position], expect_k[b, :, position], what="rotated key row in the cache")
        assert (f32(v_cache[b, :, position]) == expect_v[b, :, position]).all(), "value row is a plain copy"
    # Every other cache row is untouched.
    mask = np.ones((batch, capacity), dtype=bool)
    mask[np.arange(batch), where] = False
    assert (f32(k_cache).transpose(0, 2, 1, 3)[mask] == expect_k.transpose(0, 2, 1, 3)[mask]).all()
    assert (f32(v_cache).transpose(0, 2, 1, 3)[mask] == expect_v.transpose(0, 2, 1, 3)[mask]).all()
    # Views into one fused q|k|v row are read in place.
    fused = torch.cat([q.reshape(batch, -1), k.reshape(batch, -1), v.reshape(batch, -1)], dim=1)
    views = (fused[:, :q_heads * dim].view(batch, q_heads, dim),
             fused[:, q_heads * dim:(q_heads + kv_heads) * dim].view(batch, kv_heads, dim),
             fused[:, (q_heads + kv_heads) * dim:].view(batch, kv_heads, dim))
    assert_bit_equal(B.rope_kv_append(*views, positions, k_cache, v_cache, theta=theta), rotated, "fused-row views")


def attention_module(device, hidden=1536, heads=12, kv_heads=2, dim=128):
    def linear(seed, fan_in, fan_out):
        return blocks.QuantizedLinear.from_seed(seed, fan_in, fan_out, device)

    return blocks.Attention(linear(1, hidden, heads * dim), linear(2, hidden, kv_heads * dim),
                            linear(3, hidden, kv_heads * dim), linear(4, heads * dim, hidden), heads, kv_heads, dim, 1e6)


def filled_cache(module, batch, length, capacity, device, seed=50):
    cache = blocks.KVCache(batch, module.kv_heads, capacity, module.head_dim, device)
    cache.keys[:, :, :length] = synth.activations(seed, batch * module.kv_heads * length, module.head_dim, device,
                                                  std=0.5).reshape(batch, module.kv_heads, length, module.head_dim)
    cache.values[:, :, :length] = synth.activations(seed + 1, batch * module.kv_heads * length, module.head_dim, device,
                                                    std=0.5).reshape(batch, module.kv_heads, length, module.head_dim)
    cache.advance(length)
    return cache


def test_fused_decode_step_of_an_attention_module(cuda_device):
    """Five kernels (q|k|v, rotary + append, attention, merge, o-projection) against the module's own
    op-by-op forward (three projections, torch rotary, cache update, torch attention, o-projection) and
    against the oracle's composition of the same steps."""
    module = attention_module(cuda_device)
    batch, length, capacity = 16, 2047, 2048
    x = synth.activations(60, batch, 1536, cuda_device, std=0.5).reshape(batch, 1, 1536)
    residual = synth.activations(61, batch, 1536, cuda_device, std=0.5).reshape(batch, 1, 1536)
    cache_ref = filled_cache(module, batch, length, capacity, cuda_device)
    cache_new = filled_cache(module, batch, length, capacity, cuda_device)
    with torch.no_grad():
        expected = module(x, cache_ref)
        assert torch_lm.attention_decode_refusal(module, x, cache_new) is None
        got = torch_lm.execute_attention_decode(module, x, cache_new)
    assert cache_new.length == cache_ref.length == length + 1
    # The appended rows agree with the op-by-op path (torch rotary in fp32 vs the kernel's).
    assert_within(cache_new.keys[:, :, length], f32(cache_ref.keys[:, :, length]), what="appended key rows")
    assert_bit_equal(cache_new.values[:, :, length].contiguous(), cache_ref.values[:, :, length].contiguous(),
                     "appended value rows")
    peak = expected.float().abs().max()
    assert (got.float() - expected.float()).abs().max() <= 1e-2 * peak
    # The oracle's composition: projections (bf16-rounded weights, as the tcgen05 kernel computes them),
    # rotary, attention over the cache, output projection.
    rows = f32(x.reshape(batch, 1536))
    triple = lambda linear: (linear.weight.cpu().numpy(), f32(linear.scales), f32(linear.biases))  # noqa: E731
    q = A.qmm(rows, *triple(module.q_proj), weights="bf16").reshape(batch, 12, 128)
    k = A.qmm(rows, *triple(module.k_proj), weights="bf16").reshape(batch, 2, 128)
    positions = np.full((batch,), length)
    keys = f32(cache_ref.keys[:, :, :length + 1]).copy()
    values = f32(cache_ref.values[:, :, :length + 1]).copy()
    keys[:, :, length] = OA.rope(k, positions, 1e6)
    attended = OA.attention_decode(OA.rope(q, positions, 1e6).reshape(batch, 12, 1, 128), keys, values, 128 ** -0.5)
    oracle_out = A.qmm(attended.reshape(batch, 1536), *triple(module.o_proj), weights="bf16")
    assert_within(got.reshape(batch, 1536), oracle_out, rel=3e-3, what="fused decode step vs oracle composition")
    # With the residual in the output projection's epilogue.
    cache_res = filled_cache(module, batch, length, capacity, cuda_device)
    with torch.no_grad():
        with_residual = torch_lm.execute_attention_decode(module, x, cache_res, residual=residual)
    assert_within(with_residual.reshape(batch, 1536),
                  A.qmm(attended.reshape(batch, 1536), *triple(module.o_proj), residual=f32(residual.reshape(batch, 1536)),
                        weights="bf16"), rel=3e-3, what="fused decode step + residual")


def test_patched_attention_surfaces_and_refusals(cuda_device):
    model = blocks.random_model(seed=5, device=cuda_device, layers=1)
    original_sdpa, original_forward = blocks.scaled_dot_product_attention, blocks.Attention.forward
    tokens = torch.tensor([[1, 5, 9, 2]], device=cuda_device)
    with torch.no_grad():
        cache = model.make_cache()
        model(tokens, cache=cache)
        reference = model(torch.tensor([[7]], device=cuda_device), cache=cache).float()
        with torch_lm.apply_metile_to_torch_lm(model, attention=True, rms_norm=False, graph_fusion=False,
                                               quantized_mlp=False) as patch:
            assert blocks.scaled_dot_product_attention._metile_original is original_sdpa
            assert blocks.Attention.forward._metile_original is original_forward
            cache = model.make_cache()
            model(tokens, cache=cache)  # prefill: the model's own path, no refusal recorded for it
            out = model(torch.tensor([[7]], device=cuda_device), cache=cache).float()
            assert not patch.refusals, patch.refusals
            # A cache without room is refused at call time and served by the original forward.
            full = model.make_cache(capacity=5)
            model(tokens, cache=full)
            model(torch.tensor([[7]], device=cuda_device), cache=full)
            with pytest.raises(ValueError):
                model(torch.tensor([[7]], device=cuda_device), cache=full)  # the model's own capacity check
            assert "attention" in patch.refusals
    assert blocks.scaled_dot_product_attention is original_sdpa and blocks.Attention.forward is original_forward
    peak = reference.abs().max()
    assert (out - reference).abs().max() <= 2e-2 * peak
