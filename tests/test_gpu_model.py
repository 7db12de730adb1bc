"""GPU tests at model level: `compile` on a seeded random-init decoder-only model with 4-bit
projections, and one Qwen2.5-1.5B-shaped decoder block (hidden 1536, 12 query / 2 kv heads of 128,
intermediate 8960, RoPE theta 1e6, eps 1e-6) in prefill and 16-row decode."""

import pytest
import torch

import metile_b200
from metile_b200 import synth
from metile_b200.integrations import blocks, torch_lm
from tests.helpers import assert_bit_equal

pytestmark = pytest.mark.gpu


def test_compile_verifies_a_random_model_and_reports(cuda_device):
    model = blocks.random_model(seed=3, device=cuda_device)
    tokens = torch.tensor([[1, 5, 9, 2, 7, 3, 8, 4]], device=cuda_device)
    with torch.no_grad():
        before = model(tokens).float()
    # Exact comparison: the fused MLP keeps fp32 intermediates, the unpatched model rounds each
    # projection to bf16 first, so at tolerance 0 the report must decline rather than keep silently.
    strict = metile_b200.compile(model, tolerance=0.0)
    try:
        text = str(strict)
        assert "meTile on TinyCausalLM" in text
        for feature in strict.features:
            assert feature in ("attention", "rms_norm", "graph_fusion", "quantized_mlp")
        if "quantized_mlp" not in strict.features:
            assert "quantized_mlp" in strict.declined or "combined" in strict.declined
    finally:
        strict.restore()
    relaxed = metile_b200.compile(model, tolerance=2e-2)
    try:
        assert relaxed and relaxed.verified is True
        assert "quantized_mlp" in relaxed.features and "graph_fusion" in relaxed.features
        assert "block" in relaxed.surfaces and "mlp" in relaxed.surfaces and "self_attn" in relaxed.surfaces
        assert "attention" in relaxed.features
        assert relaxed.relative is not None and relaxed.relative <= 2e-2
        with torch.no_grad():
            after = model(tokens).float()
        peak = before.abs().max()
        assert (after - before).abs().max() <= 2e-2 * peak
    finally:
        relaxed.restore()
    with torch.no_grad():
        assert_bit_equal(model(tokens), before.to(torch.bfloat16) if before.dtype != torch.bfloat16 else before)


def test_patch_restores_every_class(cuda_device):
    model = blocks.random_model(seed=4, device=cuda_device, layers=1)
    originals = (blocks.DecoderBlock.forward, blocks.GatedMLP.forward, blocks.RMSNorm.forward,
                 blocks.Attention.forward, blocks.scaled_dot_product_attention)
    with torch_lm.apply_metile_to_torch_lm(model, attention=True) as patch:
        assert blocks.DecoderBlock.forward._metile_original is originals[0]
        assert len(patch.replacements) == 5
    assert (blocks.DecoderBlock.forward, blocks.GatedMLP.forward, blocks.RMSNorm.forward, blocks.Attention.forward,
            blocks.scaled_dot_product_attention) == originals


def qwen_block(device):
    hidden, inter, heads, kv_heads, head_dim = 1536, 8960, 12, 2, 128

    def linear(seed, fan_in, fan_out):
        return blocks.QuantizedLinear.from_seed(seed, fan_in, fan_out, device)

    attention = blocks.Attention(linear(1, hidden, heads * head_dim), linear(2, hidden, kv_heads * head_dim),
                                 linear(3, hidden, kv_heads * head_dim), linear(4, heads * head_dim, hidden), heads,
                                 kv_heads, head_dim, 1e6)
    mlp = blocks.GatedMLP(linear(5, hidden, inter), linear(6, hidden, inter), linear(7, inter, hidden))
    block = blocks.DecoderBlock(blocks.RMSNorm(synth.norm_weight(8, hidden, device), 1e-6), attention,
                                blocks.RMSNorm(synth.norm_weight(9, hidden, device), 1e-6), mlp)
    return block, hidden


def block_cache(block, batch, length, capacity, device, seed):
    attention = block.self_attn
    cache = blocks.KVCache(batch, attention.kv_heads, capacity, attention.head_dim, device)
    shape = (batch, attention.kv_heads, length, attention.head_dim)
    cache.keys[:, :, :length] = synth.activations(seed, batch * attention.kv_heads * length, attention.head_dim,
                                                  device, std=0.5).reshape(shape)
    cache.values[:, :, :length] = synth.activations(seed + 1, batch * attention.kv_heads * length,
                                                    attention.head_dim, device, std=0.5).reshape(shape)
    cache.advance(length)
    return cache


def test_qwen_block_prefill_and_decode_patched_against_unpatched(cuda_device):
    """One Qwen2.5-1.5B-shaped decoder block, patched vs unpatched: prefill of 512 tokens, then a 16-row
    decode step at KV length 2048 (16 sequences, one new token each).  The patched decode step is
    kernels only: RMSNorm, fused q|k|v, rotary + append, attention (+ merge), o-projection + residual,
    RMSNorm, the INT4 MLP.  (The pieces are checked against the oracle in tests/test_gpu_configs.py.)"""
    block, hidden = qwen_block(cuda_device)
    model = torch.nn.Module()
    model.layers = torch.nn.ModuleList([block])
    prefill = synth.activations(1, 512, hidden, cuda_device, std=0.5).reshape(1, 512, hidden)
    decode = synth.activations(2, 16, hidden, cuda_device, std=0.5).reshape(16, 1, hidden)
    with torch.no_grad():
        ref_prefill = block(prefill, blocks.KVCache(1, 2, 512, 128, cuda_device))
        ref_decode = block(decode, block_cache(block, 16, 2047, 2048, cuda_device, 3))
        with torch_lm.apply_metile_to_torch_lm(model, attention=True) as patch:
            out_prefill = block(prefill, blocks.KVCache(1, 2, 512, 128, cuda_device))
            out_decode = block(decode, block_cache(block, 16, 2047, 2048, cuda_device, 3))
            assert not patch.refusals, patch.refusals
            again = block(decode, block_cache(block, 16, 2047, 2048, cuda_device, 3))
    for out, ref in ((out_prefill, ref_prefill), (out_decode, ref_decode)):
        assert out.shape == ref.shape and torch.isfinite(out.float()).all()
        peak = ref.float().abs().max()
        assert (out.float() - ref.float()).abs().max() <= 1e-2 * peak
    assert_bit_equal(again, out_decode, "patched decode step is repeatable")
