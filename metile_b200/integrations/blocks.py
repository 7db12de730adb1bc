"""torch modules that carry MLX-format INT4 weights: the structural targets of the patcher.

They mirror what the reference patches inside MLX-LM models (metile/integrations/mlx_lm.py):
`QuantizedLinear` (MLX's nn.QuantizedLinear: weight / scales / biases, group_size, bits, mode),
an RMSNorm, a gated MLP with gate_proj / up_proj / down_proj, a decoder block with
input_layernorm / self_attn / post_attention_layernorm / mlp, and a small causal LM used to verify
logits before and after patching.  Every INT4 projection runs the CUDA kernels; none has a CPU
path.  The UNPATCHED forward of each module is the op-by-op form native MLX computes
(metile/backends/mlx_quantized.py:883-917: each projection rounded to bf16, then silu(gate)*up,
then down, then the residual add), so that patching reproduces the reference's situation: the
fused path keeps fp32 intermediates and can differ from the op-by-op path by rounding.
"""

from __future__ import annotations

import math

import torch
from torch import nn

from .. import backends


class QuantizedLinear(nn.Module):
    """y = x @ dequant(weight)^T (+ bias) with MLX affine INT4 weights."""

    def __init__(self, weight, scales, biases, *, group_size=64, bits=4, bias=None, mode="affine"):
        super().__init__()
        self.register_buffer("weight", weight)
        self.register_buffer("scales", scales)
        self.register_buffer("biases", biases)
        self.group_size = group_size
        self.bits = bits
        self.mode = mode
        if bias is not None:
            self.register_buffer("bias", bias)
        else:
            self.bias = None

    @property
    def in_features(self):
        return self.weight.shape[1] * 32 // self.bits

    @property
    def out_features(self):
        return self.weight.shape[0]

    @classmethod
    def from_seed(cls, seed, in_features, out_features, device="cpu"):
        from .. import synth

        return cls(*synth.affine_weight(seed, out_features, in_features, device))

    def forward(self, values):
        out = backends.mlx_affine_qmv(values, self.weight, self.scales, self.biases,
                                      group_size=self.group_size, bits=self.bits)
        return out if self.bias is None else out + self.bias


class QuantizedEmbedding(nn.Module):
    """Token embedding stored as affine INT4 rows (MLX's nn.QuantizedEmbedding: weight uint32
    [V, H/8], scales / biases [V, H/64]).  A lookup gathers the packed rows of the tokens and
    dequantises just those (w = scale * q + bias in fp32, one rounding to the scales' dtype);
    `as_linear()` serves the same triple as the tied output projection."""

    def __init__(self, weight, scales, biases, *, group_size=64, bits=4):
        super().__init__()
        self.register_buffer("weight", weight)
        self.register_buffer("scales", scales)
        self.register_buffer("biases", biases)
        self.group_size, self.bits, self.mode = group_size, bits, "affine"

    def forward(self, tokens):
        flat = tokens.reshape(-1)
        packed = self.weight.view(torch.int32)[flat]                       # [T, H/8]
        shifts = torch.arange(0, 32, 4, device=packed.device, dtype=torch.int32)
        q = ((packed[..., None] >> shifts) & 15).reshape(flat.shape[0], -1).float()   # [T, H]
        scales = self.scales[flat].float().repeat_interleave(self.group_size, dim=1)
        biases = self.biases[flat].float().repeat_interleave(self.group_size, dim=1)
        return (q * scales + biases).to(self.scales.dtype).reshape(*tokens.shape, -1)

    def as_linear(self):
        return QuantizedLinear(self.weight, self.scales, self.biases, group_size=self.group_size, bits=self.bits)


class RMSNorm(nn.Module):
    def __init__(self, weight, eps=1e-6):
        super().__init__()
        self.register_buffer("weight", weight)
        self.eps = eps

    def forward(self, values):
        # Op-by-op reference form in torch (float32 inside, one rounding at the end).
        v = values.float()
        return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight.float()).to(values.dtype)


class GatedMLP(nn.Module):
    """down_proj(silu(gate_proj(x)) * up_proj(x)), each op rounded to the activation dtype."""

    def __init__(self, gate_proj, up_proj, down_proj):
        super().__init__()
        self.gate_proj, self.up_proj, self.down_proj = gate_proj, up_proj, down_proj

    def forward(self, values):
        return self.down_proj(nn.functional.silu(self.gate_proj(values)) * self.up_proj(values))


def _rope(values, positions, theta):
    """Rotary embedding over the last axis (half-split form); values [B, heads, T, D], positions [T]
    or [B, T]."""
    dim = values.shape[-1]
    inverse = 1.0 / (theta ** (torch.arange(0, dim, 2, device=values.device, dtype=torch.float32) / dim))
    angles = positions.float()[..., None] * inverse
    if angles.ndim == 2:
        angles = angles[None]
    cos, sin = angles.cos()[:, None], angles.sin()[:, None]
    first, second = values.float()[..., : dim // 2], values.float()[..., dim // 2:]
    return torch.cat([first * cos - second * sin, second * cos + first * sin], dim=-1).to(values.dtype)


class KVCache:
    """Append-only key/value cache with room for `capacity` tokens per head, updated in place.

    The MLX-LM cache the reference's models use (`KVCache.update_and_fetch`) grows by concatenation;
    here the storage is allocated once as [batch, kv_heads, capacity, head_dim] and a step writes its
    rows at `length`, so a decode step moves only the new token's bytes."""

    def __init__(self, batch, kv_heads, capacity, head_dim, device, dtype=torch.bfloat16):
        self.keys = torch.zeros((batch, kv_heads, capacity, head_dim), dtype=dtype, device=device)
        self.values = torch.zeros_like(self.keys)
        self.length = 0
        self.positions = torch.zeros((batch,), dtype=torch.int32, device=device)

    @property
    def capacity(self):
        return self.keys.shape[2]

    def update_and_fetch(self, keys, values):
        """Write keys / values [B, H, T, D] at the current length; return views of all tokens so far."""
        steps = keys.shape[2]
        if self.length + steps > self.capacity:
            raise ValueError("KV cache capacity exceeded")
        self.keys[:, :, self.length:self.length + steps] = keys
        self.values[:, :, self.length:self.length + steps] = values
        self.advance(steps)
        return self.keys[:, :, :self.length], self.values[:, :, :self.length]

    def advance(self, steps=1):
        # The device-side count is incremented, not overwritten with the host's number, so that a
        # captured CUDA graph of a decode step advances it on every replay.
        self.length += steps
        self.positions.add_(steps)

    def reset(self, length=0):
        """Forget everything after the first `length` tokens (host and device counts together)."""
        self.length = int(length)
        self.positions.fill_(self.length)


def scaled_dot_product_attention(queries, keys, values, cache, scale, mask=None):
    """The attention primitive every Attention module here calls; the patcher replaces THIS module
    attribute (the reference replaces mlx_lm.models.base.scaled_dot_product_attention the same way,
    metile/integrations/mlx_lm.py:4607-4655).  queries [B, Hq, T, D], keys / values [B, Hkv, N, D]."""
    del cache
    causal = mask == "causal"
    return nn.functional.scaled_dot_product_attention(
        queries, keys, values, scale=scale, is_causal=causal, enable_gqa=queries.shape[1] != keys.shape[1])


class Attention(nn.Module):
    """Grouped-query attention over INT4 q/k/v/o projections with RoPE and an in-place KV cache."""

    def __init__(self, q_proj, k_proj, v_proj, o_proj, heads, kv_heads, head_dim, rope_theta=1e6):
        super().__init__()
        self.q_proj, self.k_proj, self.v_proj, self.o_proj = q_proj, k_proj, v_proj, o_proj
        self.heads, self.kv_heads, self.head_dim, self.rope_theta = heads, kv_heads, head_dim, rope_theta
        self.scale = head_dim ** -0.5

    def forward(self, values, cache=None):
        batch, steps, _ = values.shape
        q = self.q_proj(values).view(batch, steps, self.heads, self.head_dim).transpose(1, 2)
        k = self.k_proj(values).view(batch, steps, self.kv_heads, self.head_dim).transpose(1, 2)
        v = self.v_proj(values).view(batch, steps, self.kv_heads, self.head_dim).transpose(1, 2)
        offset = 0 if cache is None else cache.length
        if steps > 1 and offset > 0:
            raise ValueError("multi-token continuation is not supported by this harness")
        positions = torch.arange(offset, offset + steps, device=values.device)
        q, k = _rope(q, positions, self.rope_theta), _rope(k, positions, self.rope_theta)
        if cache is not None:
            k, v = cache.update_and_fetch(k, v)
        out = scaled_dot_product_attention(q, k, v, cache, self.scale, "causal" if steps > 1 else None)
        return self.o_proj(out.transpose(1, 2).reshape(batch, steps, self.heads * self.head_dim))


class DecoderBlock(nn.Module):
    """Pre-norm decoder block: x + attn(norm(x)), then h + mlp(norm(h))."""

    def __init__(self, input_layernorm, self_attn, post_attention_layernorm, mlp):
        super().__init__()
        self.input_layernorm, self.self_attn = input_layernorm, self_attn
        self.post_attention_layernorm, self.mlp = post_attention_layernorm, mlp

    def forward(self, values, cache=None):
        hidden = values + self.self_attn(self.input_layernorm(values), cache)
        return hidden + self.mlp(self.post_attention_layernorm(hidden))


class TinyCausalLM(nn.Module):
    """Embedding, a stack of DecoderBlocks, final norm and an INT4 lm_head; random initialisation."""

    def __init__(self, embed, layers, norm, lm_head, vocab_size):
        super().__init__()
        self.embed_tokens = embed
        self.layers = nn.ModuleList(layers)
        self.norm = norm
        self.lm_head = lm_head
        self.vocab_size = vocab_size

    def make_cache(self, batch=1, capacity=64):
        caches = []
        for layer in self.layers:
            attention = layer.self_attn
            caches.append(KVCache(batch, attention.kv_heads, capacity, attention.head_dim,
                                  attention.q_proj.weight.device))
        return caches

    def forward(self, tokens, cache=None):
        hidden = self.embed_tokens(tokens)
        for index, layer in enumerate(self.layers):
            hidden = layer(hidden, None if cache is None else cache[index])
        return self.lm_head(self.norm(hidden))


def random_model(seed=0, *, hidden=256, intermediate=512, heads=4, kv_heads=2, head_dim=64, layers=2, vocab=512,
                 rope_theta=1e6, eps=1e-6, device="cuda", quantized_embedding=False, tie_word_embeddings=False):
    """A seeded random-init decoder-only model in the Qwen2.5 / Llama layout with 4-bit projections
    (and, when asked, a 4-bit embedding, optionally tied to the output projection)."""
    from .. import synth

    def linear(offset, fan_in, fan_out):
        return QuantizedLinear.from_seed(seed * 1000 + offset, fan_in, fan_out, device)

    blocks = []
    for index in range(layers):
        base = 10 * index
        attention = Attention(linear(base + 1, hidden, heads * head_dim), linear(base + 2, hidden, kv_heads * head_dim),
                              linear(base + 3, hidden, kv_heads * head_dim), linear(base + 4, heads * head_dim, hidden),
                              heads, kv_heads, head_dim, rope_theta)
        mlp = GatedMLP(linear(base + 5, hidden, intermediate), linear(base + 6, hidden, intermediate),
                       linear(base + 7, intermediate, hidden))
        blocks.append(DecoderBlock(RMSNorm(synth.norm_weight(seed * 1000 + base + 8, hidden, device), eps), attention,
                                   RMSNorm(synth.norm_weight(seed * 1000 + base + 9, hidden, device), eps), mlp))
    generator = torch.Generator().manual_seed(seed * 1000 + 999)
    table = (torch.randn((vocab, hidden), generator=generator) / math.sqrt(hidden) * 4).to(torch.bfloat16)
    if quantized_embedding or tie_word_embeddings:
        from . import checkpoint

        embed = QuantizedEmbedding(*(t.to(device) for t in checkpoint.quantize_affine(table)))
    else:
        embed = nn.Embedding.from_pretrained(table.to(device), freeze=True)
    head = embed.as_linear() if tie_word_embeddings else linear(997, hidden, vocab)
    return TinyCausalLM(embed, blocks, RMSNorm(synth.norm_weight(seed * 1000 + 998, hidden, device), eps), head, vocab)
