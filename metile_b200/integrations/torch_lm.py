"""Reversible patching of torch models whose layers carry MLX-format INT4 weights.

torch-side equivalent of the reference's MLX-LM patcher (metile/integrations/mlx_lm.py):
  * apply_metile_to_torch_lm(...) -> TorchPatch       (apply_metile_to_mlx_lm, :4500-4699)
  * TorchPatch.restore() / context manager             (MLXPatch, :305-333)
  * class-level replacement of `forward`, the replacement carrying `_metile_original`
    (:3791, :3927), admitted by structure (:186-237) and gated per call (:3805-3834)
  * fused decoder block: attention, fused add+RMSNorm, then down(swiglu(norm)) + hidden
    (:3689-3785, decision table in the same function)
  * decode attention behind the model modules' `scaled_dot_product_attention` attribute
    (:4607-4655), admitted per call by the reference's shape rule (:3558-3573); and, beyond the
    reference, the whole decode step of an attention module as five kernels (fused q|k|v projection,
    rotary embedding + in-place cache append, split-KV attention + merge, output projection with the
    residual in its epilogue)

What differs on purpose: there is no tournament and no silent rerouting to a "native wins"
choice.  A call the kernels cannot serve (wrong format, dtype, device, an additive bias) runs the
module's ORIGINAL forward, and the reason is recorded once in `TorchPatch.refusals`, which
`metile_b200.compile` copies into its report.
"""

from __future__ import annotations

import sys
import weakref
from dataclasses import dataclass, field

import torch

from .. import backends

FEATURES = ("attention", "rms_norm", "graph_fusion", "quantized_mlp")
_GATED_MLP_ATTRIBUTES = ("gate_proj", "up_proj", "down_proj")
_FUSED_BLOCK_ATTRIBUTES = ("input_layernorm", "post_attention_layernorm", "mlp")
_ATTENTION_ATTRIBUTES = ("q_proj", "k_proj", "v_proj", "o_proj")


@dataclass
class TorchPatch:
    """A reversible set of class-level `forward` replacements."""

    replacements: list = field(default_factory=list)
    refusals: dict = field(default_factory=dict)

    def restore(self):
        for owner, name, original in reversed(self.replacements):
            setattr(owner, name, original)
        self.replacements.clear()

    def __enter__(self):
        return self

    def __exit__(self, *_):
        self.restore()

    def refuse(self, surface, reason):
        self.refusals.setdefault(surface, reason)


def _model_layers(model):
    inner = getattr(model, "model", model)
    layers = getattr(inner, "layers", None)
    return list(layers) if layers is not None else []


def _own_forward(cls):
    """The `forward` a class (or one of its bases other than nn.Module) defines itself, else None.

    nn.Module's own `forward` is a placeholder that raises; a class that inherits only that one has
    nothing to replace (the reference makes the same point about `__call__`,
    metile/integrations/mlx_lm.py:195-214)."""
    for klass in cls.__mro__:
        if klass is torch.nn.Module:
            break
        if "forward" in vars(klass):
            return vars(klass)["forward"]
    return None


def _forward_source(cls):
    import inspect

    function = _own_forward(cls)
    if function is None:
        return None
    try:
        return inspect.getsource(function)
    except (OSError, TypeError):
        return None


def _structurally_matches(cls, required):
    """Whether `cls` is a candidate for the replacement that needs the attributes `required`.

    The class must define its own forward, and every required name must be visible on the class: as a
    class attribute or annotation, or -- torch modules bind their parts in __init__ -- in the source of
    that forward.  So an attention class is not taken for a gated MLP, nor an MLP for a decoder block.
    A structural match only admits a candidate; `compile` still verifies the logits."""
    if _own_forward(cls) is None:
        return False
    annotations = getattr(cls, "__annotations__", {})
    if all(hasattr(cls, name) or name in annotations for name in required):
        return True
    source = _forward_source(cls)
    return source is not None and all(name in source for name in required)


def _has_parts(module, required):
    return all(getattr(module, name, None) is not None for name in required)


def _is_affine_int4(linear):
    return (
        getattr(linear, "mode", None) == "affine"
        and getattr(linear, "group_size", None) == 64
        and getattr(linear, "bits", None) == 4
        and getattr(linear, "weight", None) is not None
        and getattr(linear, "scales", None) is not None
        and getattr(linear, "biases", None) is not None
    )


def quantized_mlp_refusal(module, values):
    """None when the fused INT4 MLP can serve this call, else the reason it cannot.

    Mirrors _supports_quantized_mlp / _supports_quantized_residual_mlp of the reference
    (metile/integrations/mlx_lm.py:3805-3834): three affine 4-bit group-64 projections with
    quantisation biases and no additive bias; activations in the kernels' dtype (bfloat16 here,
    float16 there) on a CUDA device.
    """
    for name in _GATED_MLP_ATTRIBUTES:
        linear = getattr(module, name, None)
        if linear is None:
            return f"{name} is missing"
        if not _is_affine_int4(linear):
            return f"{name} is not an affine 4-bit group-64 quantized projection"
        if getattr(linear, "bias", None) is not None:
            return f"{name} has an additive bias"
    if values.dtype != torch.bfloat16:
        return f"activations are {values.dtype}, the kernels take bfloat16"
    if not values.is_cuda:
        return "activations are not on a CUDA device"
    gate, up, down = module.gate_proj, module.up_proj, module.down_proj
    if gate.weight.shape != up.weight.shape or down.weight.shape[0] != values.shape[-1]:
        return "projection shapes do not form gate|up -> down"
    return None


_executor_cache = weakref.WeakKeyDictionary()


def execute_quantized_mlp(module, values, residual=None):
    """down(swiglu(values)) (+ residual) through one bound executor per module.

    The executor is cached per module and dropped with it (the reference keys its cache by module
    id with weakref eviction, metile/integrations/mlx_lm.py:3854-3885)."""
    execute = _executor_cache.get(module)
    if execute is None:
        gate, up, down = module.gate_proj, module.up_proj, module.down_proj
        execute = backends.mlx_affine_mlp_executor(
            values, gate.weight, gate.scales, gate.biases, up.weight, up.scales, up.biases, down.weight,
            down.scales, down.biases, None)
        _executor_cache[module] = execute
    return execute(values, residual)


_qkv_cache = weakref.WeakKeyDictionary()


def attention_decode_refusal(module, values, cache):
    """None when the five-kernel decode step can serve this call of an attention module, else why not:
    one new token per sequence, an in-place cache with room left, four affine 4-bit projections
    without additive bias, bfloat16 activations on CUDA, and a head layout the kernels take."""
    if values.ndim != 3 or values.shape[1] != 1:
        return "not a single-token decode step"
    if cache is None or not all(hasattr(cache, name) for name in ("keys", "values", "length", "positions", "advance")):
        return "no in-place KV cache"
    if cache.length < 1 or cache.length >= cache.keys.shape[2]:
        return "the cache is empty or full"
    for name in _ATTENTION_ATTRIBUTES:
        linear = getattr(module, name, None)
        if linear is None or not _is_affine_int4(linear):
            return f"{name} is not an affine 4-bit group-64 quantized projection"
        if getattr(linear, "bias", None) is not None:
            return f"{name} has an additive bias"
    heads, kv_heads, dim = (getattr(module, name, None) for name in ("heads", "kv_heads", "head_dim"))
    if not heads or not kv_heads or dim not in (64, 128) or heads % kv_heads or heads // kv_heads > 8:
        return "head layout outside what the decode kernel serves"
    if getattr(module, "rope_theta", None) is None:
        return "no rotary base"
    if values.dtype != torch.bfloat16 or not values.is_cuda:
        return "activations are not bfloat16 on a CUDA device"
    if values.shape[0] != cache.keys.shape[0]:
        return "batch does not match the cache"
    return None


def _fused_qkv(module):
    """The q, k and v triples concatenated along the output axis, built once per module: one
    projection launch reads the activations once and writes one q|k|v row per sequence."""
    fused = _qkv_cache.get(module)
    if fused is None:
        parts = (module.q_proj, module.k_proj, module.v_proj)
        fused = tuple(torch.cat([getattr(linear, name) for linear in parts], dim=0).contiguous()
                      for name in ("weight", "scales", "biases"))
        _qkv_cache[module] = fused
    return fused


def execute_attention_decode(module, values, cache, residual=None):
    """One decode step of an attention module without a framework op between its kernels:
    fused q|k|v projection, rotary embedding + cache append, attention over the cache, output
    projection (+ residual, added to the un-rounded sum).  values [B, 1, H]; returns [B, 1, H]."""
    batch = values.shape[0]
    heads, kv_heads, dim = module.heads, module.kv_heads, module.head_dim
    rows = values.reshape(batch, values.shape[-1])
    qkv = backends.mlx_affine_qmv(rows, *_fused_qkv(module))
    q = qkv[:, :heads * dim].view(batch, heads, dim)
    k = qkv[:, heads * dim:(heads + kv_heads) * dim].view(batch, kv_heads, dim)
    v = qkv[:, (heads + kv_heads) * dim:].view(batch, kv_heads, dim)
    rotated = backends.rope_kv_append(q, k, v, cache.positions, cache.keys, cache.values, theta=module.rope_theta)
    cache.advance(1)
    scale = getattr(module, "scale", dim ** -0.5)
    # The whole cache with the per-sequence lengths on the device (not a slice cut at the host's count):
    # the same 128-token splits are merged either way, and nothing of the step depends on a host number,
    # so a captured CUDA graph of it stays valid as the sequences grow.
    attended = backends.mlx_attention_decode(rotated.view(batch, heads, 1, dim), cache.keys, cache.values,
                                             scale=scale, lengths=cache.positions)
    attended = attended.view(batch, heads * dim)
    o = module.o_proj
    if residual is None:
        out = backends.mlx_affine_qmv(attended, o.weight, o.scales, o.biases)
    else:
        out = backends.mlx_affine_residual_qmv(attended, o.weight, o.scales, o.biases,
                                               residual.reshape(batch, residual.shape[-1]))
    return out.view(values.shape)


def _replace_forward(patch, cls, make_replacement):
    original = cls.forward
    if getattr(original, "_metile_original", None) is not None:
        return False
    replacement = make_replacement(original)
    replacement._metile_original = original
    patch.replacements.append((cls, "forward", original))
    cls.forward = replacement
    return True


def _patch_quantized_mlp(model, patch, min_rows=1, max_rows=None):
    if min_rows < 1:
        raise ValueError("quantized MLP minimum rows must be positive")
    if max_rows is not None and max_rows < min_rows:
        raise ValueError("quantized MLP maximum rows must not be smaller than its minimum")
    classes = [type(layer.mlp) for layer in _model_layers(model) if getattr(layer, "mlp", None) is not None]
    for mlp_class in dict.fromkeys(classes):
        if not _structurally_matches(mlp_class, _GATED_MLP_ATTRIBUTES):
            continue

        def make(original):
            def replacement(self, values):
                rows = values.numel() // values.shape[-1]
                if rows < min_rows or (max_rows is not None and rows > max_rows):
                    return original(self, values)
                reason = quantized_mlp_refusal(self, values) if _has_parts(self, _GATED_MLP_ATTRIBUTES) \
                    else "the module lacks gate_proj / up_proj / down_proj"
                if reason is not None:
                    patch.refuse("quantized_mlp", reason)
                    return original(self, values)
                return execute_quantized_mlp(self, values)

            return replacement

        _replace_forward(patch, mlp_class, make)


def _norm_eps(norm):
    for name in ("eps", "variance_epsilon"):
        if hasattr(norm, name):
            return float(getattr(norm, name))
    return None


def _patch_rms_norm(model, patch):
    classes = []
    for layer in _model_layers(model):
        for name in ("input_layernorm", "post_attention_layernorm"):
            norm = getattr(layer, name, None)
            if norm is not None:
                classes.append(type(norm))
    final = getattr(getattr(model, "model", model), "norm", None)
    if final is not None:
        classes.append(type(final))
    for norm_class in dict.fromkeys(classes):
        if not _structurally_matches(norm_class, ("weight",)):
            continue

        def make(original):
            def replacement(self, values):
                eps = _norm_eps(self)
                weight = getattr(self, "weight", None)
                if eps is None or weight is None or values.dtype != torch.bfloat16 or not values.is_cuda \
                        or weight.dtype != values.dtype:
                    patch.refuse("rms_norm", "the norm has no weight/eps or is not bfloat16 on CUDA")
                    return original(self, values)
                return backends.mlx_rms_norm(values, weight, eps)

            return replacement

        _replace_forward(patch, norm_class, make)


def _patch_attention(model, patch):
    """Decode attention.  Two surfaces, as far as the model offers them:
    (1) the `scaled_dot_product_attention` attribute of the module that defines the model's attention
        class is replaced by a function that serves single-row, unmasked calls with the decode kernel
        and passes everything else to the original (the reference's scheme);
    (2) attention classes with q/k/v/o projections and an in-place cache run their decode steps as five
        kernels (execute_attention_decode); prefill and unsupported calls run the original forward."""
    classes = [type(layer.self_attn) for layer in _model_layers(model) if getattr(layer, "self_attn", None) is not None]
    before = len(patch.replacements)
    for attention_class in dict.fromkeys(classes):
        home = sys.modules.get(attention_class.__module__)
        original_sdpa = getattr(home, "scaled_dot_product_attention", None)
        if original_sdpa is not None and getattr(original_sdpa, "_metile_original", None) is None:

            def metile_scaled_dot_product_attention(queries, keys, values, cache, scale, mask=None,
                                                    _original=original_sdpa):
                reason = backends.supports_attention_decode(queries, keys, values, mask)
                if reason is None:
                    return backends.mlx_attention_decode(queries, keys, values, scale=scale)
                if queries.ndim == 4 and queries.shape[2] == 1:
                    patch.refuse("attention", reason)
                return _original(queries, keys, values, cache, scale, mask)

            metile_scaled_dot_product_attention._metile_original = original_sdpa
            patch.replacements.append((home, "scaled_dot_product_attention", original_sdpa))
            home.scaled_dot_product_attention = metile_scaled_dot_product_attention

        if not _structurally_matches(attention_class, _ATTENTION_ATTRIBUTES):
            continue

        def make(original):
            def replacement(self, values, cache=None, *args, **kwargs):
                if args or kwargs or values.ndim != 3 or values.shape[1] != 1:
                    return original(self, values, cache, *args, **kwargs)  # prefill: the model's own path
                reason = attention_decode_refusal(self, values, cache)
                if reason is not None:
                    patch.refuse("attention", reason)
                    return original(self, values, cache)
                return execute_attention_decode(self, values, cache)

            return replacement

        _replace_forward(patch, attention_class, make)
    if len(patch.replacements) == before:
        patch.refuse("attention", "the model exposes no attention surface that can be replaced")


def _patch_graph_fusion(model, patch, quantized_mlp):
    classes = [type(layer) for layer in _model_layers(model)]
    for block_class in dict.fromkeys(classes):
        if not _structurally_matches(block_class, _FUSED_BLOCK_ATTRIBUTES):
            continue

        def make(original):
            def replacement(self, values, *args, **kwargs):
                attention = getattr(self, "self_attn", None)
                post = getattr(self, "post_attention_layernorm", None)
                eps = _norm_eps(post) if post is not None else None
                if attention is None or not _has_parts(self, _FUSED_BLOCK_ATTRIBUTES) or eps is None:
                    patch.refuse("graph_fusion", "the block does not bind self_attn and two RMSNorms with eps")
                    return original(self, values, *args, **kwargs)
                if values.dtype != torch.bfloat16 or not values.is_cuda:
                    patch.refuse("graph_fusion", "activations are not bfloat16 on a CUDA device")
                    return original(self, values, *args, **kwargs)
                normed_input = self.input_layernorm(values)
                cache = args[0] if args else kwargs.get("cache")
                fused_attention = (
                    getattr(type(attention).forward, "_metile_original", None) is not None
                    and len(args) <= 1 and set(kwargs) <= {"cache"}
                    and _has_parts(attention, _ATTENTION_ATTRIBUTES)
                    and attention_decode_refusal(attention, normed_input, cache) is None)
                if fused_attention:
                    # The residual rides in the output projection's epilogue (added to the un-rounded
                    # sum), so only the norm is left of the add + RMSNorm.
                    hidden = execute_attention_decode(attention, normed_input, cache, residual=values)
                    normalized = backends.mlx_rms_norm(hidden, post.weight, eps)
                else:
                    attended = attention(normed_input, *args, **kwargs)
                    hidden, normalized = backends.mlx_add_rms_norm(values, attended, post.weight, eps)
                if quantized_mlp:
                    reason = quantized_mlp_refusal(self.mlp, normalized)
                    if reason is None:
                        return execute_quantized_mlp(self.mlp, normalized, hidden)
                    patch.refuse("quantized_mlp", reason)
                return hidden + self.mlp(normalized)

            return replacement

        _replace_forward(patch, block_class, make)


def apply_metile_to_torch_lm(model=None, *, attention=False, rms_norm=True, graph_fusion=True,
                             quantized_mlp=True, quantized_mlp_min_rows=1, quantized_mlp_max_rows=None):
    """Patch the classes `model`'s layers use and return the reversible handle.

    attention: single-row, unmasked attention calls run the decode-attention kernel; attention modules
        with INT4 q/k/v/o projections and an in-place cache run a whole decode step as five kernels.
    rms_norm: RMSNorm modules run the CUDA RMSNorm.
    graph_fusion: decoder blocks run attention, then the fused residual add + RMSNorm, then (with
        quantized_mlp) the fused INT4 MLP with the residual folded into the down projection.
    quantized_mlp: gated MLP modules run gate|up SwiGLU -> down as two kernels behind one call.
    """
    if model is None:
        raise ValueError("apply_metile_to_torch_lm needs the model whose classes are to be patched")
    # Every argument is checked before the first class is touched: an exception must not leave a
    # half-applied patch behind with no handle to undo it.
    if quantized_mlp_min_rows < 1:
        raise ValueError("quantized MLP minimum rows must be positive")
    if quantized_mlp_max_rows is not None and quantized_mlp_max_rows < quantized_mlp_min_rows:
        raise ValueError("quantized MLP maximum rows must not be smaller than its minimum")
    patch = TorchPatch()
    if attention:
        _patch_attention(model, patch)
    if graph_fusion:
        _patch_graph_fusion(model, patch, quantized_mlp)
    if quantized_mlp:
        _patch_quantized_mlp(model, patch, quantized_mlp_min_rows, quantized_mlp_max_rows)
    if rms_norm:
        _patch_rms_norm(model, patch)
    return patch
