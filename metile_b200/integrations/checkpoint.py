"""MLX-community 4-bit checkpoints on disk: a safetensors reader / writer and the mapping between
the checkpoint's tensor names and the torch modules of `blocks`.

The reference never parses checkpoints itself: it patches models that `mlx_lm.load` has built, whose
`nn.QuantizedLinear` layers hold the `weight` (uint32 [N, K/8]) / `scales` / `biases` ([N, K/64])
triples exactly as the file stores them (metile/integrations/mlx_lm.py works on those attributes;
layout in metile/backends/mlx_quantized.py:478-480, 768-769).  Here the same triples are read from the
file and handed to the CUDA operators unchanged: no repacking, no transposition.

File format (safetensors): 8 bytes little-endian header length, a JSON header mapping each tensor
name to {"dtype", "shape", "data_offsets": [begin, end)} relative to the end of the header (plus an
optional "__metadata__" string map), then the raw little-endian tensor bytes.

Directory layout read and written: `config.json` (Llama / Qwen2 field names, with
"quantization": {"group_size": 64, "bits": 4}) and either `model.safetensors` or shards listed by
`model.safetensors.index.json` ("weight_map": name -> file).  Tensor names:
  model.embed_tokens.{weight,scales,biases}      (quantised embedding; dense: weight only)
  model.layers.<i>.self_attn.{q,k,v,o}_proj.{weight,scales,biases[,bias]}
  model.layers.<i>.mlp.{gate,up,down}_proj.{weight,scales,biases}
  model.layers.<i>.{input_layernorm,post_attention_layernorm}.weight
  model.norm.weight, lm_head.{weight,scales,biases}  (absent when tie_word_embeddings)
"""

from __future__ import annotations

import json
import os
import struct

import numpy as np
import torch

from . import blocks

_DTYPES = {
    "U32": (np.uint32, torch.uint32),
    "I32": (np.int32, torch.int32),
    "I64": (np.int64, torch.int64),
    "U8": (np.uint8, torch.uint8),
    "F32": (np.float32, torch.float32),
    "F16": (np.float16, torch.float16),
    "BF16": (np.uint16, torch.bfloat16),  # numpy has no bfloat16: carried as bit patterns
}
_NAMES = {torch_type: name for name, (_, torch_type) in _DTYPES.items()}


def read_safetensors(path):
    """{name: CPU tensor} of one .safetensors file, plus the "__metadata__" map under that key."""
    with open(path, "rb") as handle:
        prefix = handle.read(8)
        if len(prefix) != 8:
            raise ValueError(f"{path}: not a safetensors file (shorter than its length prefix)")
        (length,) = struct.unpack("<Q", prefix)
        size = os.path.getsize(path)
        if length > size - 8:
            raise ValueError(f"{path}: header length {length} exceeds the file")
        header = json.loads(handle.read(length).decode("utf-8"))
        payload = np.frombuffer(handle.read(), dtype=np.uint8)
    tensors = {}
    for name, entry in header.items():
        if name == "__metadata__":
            tensors[name] = dict(entry)
            continue
        if entry["dtype"] not in _DTYPES:
            raise ValueError(f"{path}: tensor {name!r} has unsupported dtype {entry['dtype']}")
        numpy_type, torch_type = _DTYPES[entry["dtype"]]
        begin, end = entry["data_offsets"]
        shape = tuple(entry["shape"])
        count = int(np.prod(shape, dtype=np.int64)) if shape else 1
        if begin < 0 or end > payload.size or end - begin != count * np.dtype(numpy_type).itemsize:
            raise ValueError(f"{path}: tensor {name!r} has inconsistent offsets {begin}:{end} for shape {shape}")
        array = payload[begin:end].view(numpy_type).reshape(shape).copy()
        tensor = torch.from_numpy(array)
        tensors[name] = tensor.view(torch.bfloat16) if torch_type is torch.bfloat16 else tensor
    return tensors


def write_safetensors(path, tensors, metadata=None):
    """Write {name: tensor} (any device) as one .safetensors file; names are stored sorted."""
    header, chunks, offset = {}, [], 0
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    for name in sorted(tensors):
        tensor = tensors[name].detach().cpu().contiguous()
        if tensor.dtype not in _NAMES:
            raise ValueError(f"tensor {name!r} has unsupported dtype {tensor.dtype}")
        raw = (tensor.view(torch.uint16) if tensor.dtype is torch.bfloat16 else tensor).numpy().tobytes()
        header[name] = {"dtype": _NAMES[tensor.dtype], "shape": list(tensor.shape), "data_offsets": [offset, offset + len(raw)]}
        chunks.append(raw)
        offset += len(raw)
    encoded = json.dumps(header, separators=(",", ":")).encode("utf-8")
    encoded += b" " * (-len(encoded) % 8)  # the payload starts 8-byte aligned
    with open(path, "wb") as handle:
        handle.write(struct.pack("<Q", len(encoded)))
        handle.write(encoded)
        for raw in chunks:
            handle.write(raw)


def read_checkpoint_tensors(directory):
    """Every tensor of a checkpoint directory: one model.safetensors, or the shards of its index."""
    index = os.path.join(directory, "model.safetensors.index.json")
    if os.path.exists(index):
        with open(index) as handle:
            weight_map = json.load(handle)["weight_map"]
        tensors = {}
        for shard in sorted(set(weight_map.values())):
            loaded = read_safetensors(os.path.join(directory, shard))
            loaded.pop("__metadata__", None)
            tensors.update(loaded)
        missing = sorted(set(weight_map) - set(tensors))
        if missing:
            raise ValueError(f"{directory}: the index names tensors no shard holds: {missing[:4]}")
        return tensors
    tensors = read_safetensors(os.path.join(directory, "model.safetensors"))
    tensors.pop("__metadata__", None)
    return tensors


def quantize_affine(weight, group_size=64, bits=4):
    """Dense [N, K] -> (uint32 [N, K/8], scales, biases [N, K/group]) by min/max per group, so that
    w ~ scale * q + bias.  For building test checkpoints; not claimed bit-identical to `mx.quantize`."""
    if bits != 4 or group_size != 64:
        raise ValueError("affine quantisation here is 4 bits, group size 64")
    from .. import synth

    rows, columns = weight.shape
    groups = weight.float().reshape(rows, columns // group_size, group_size)
    low, high = groups.amin(-1), groups.amax(-1)
    scales = ((high - low) / 15.0).clamp_min(1e-8).to(torch.bfloat16)
    biases = low.to(torch.bfloat16)
    q = ((groups - biases.float()[..., None]) / scales.float()[..., None]).round().clamp(0, 15).to(torch.int64)
    return synth.pack_nibbles(q.reshape(rows, columns)), scales, biases


def _linear_tensors(prefix, linear):
    out = {f"{prefix}.weight": linear.weight, f"{prefix}.scales": linear.scales, f"{prefix}.biases": linear.biases}
    if getattr(linear, "bias", None) is not None:
        out[f"{prefix}.bias"] = linear.bias
    return out


def model_config(model):
    """config.json content (Llama / Qwen2 field names) of a `blocks.TinyCausalLM`."""
    first = model.layers[0]
    attention = first.self_attn
    return {
        "model_type": "qwen2" if attention.q_proj.bias is not None else "llama",
        "hidden_size": attention.q_proj.in_features,
        "intermediate_size": first.mlp.gate_proj.out_features,
        "num_hidden_layers": len(model.layers),
        "num_attention_heads": attention.heads,
        "num_key_value_heads": attention.kv_heads,
        "head_dim": attention.head_dim,
        "rms_norm_eps": first.input_layernorm.eps,
        "rope_theta": attention.rope_theta,
        "vocab_size": model.vocab_size,
        "tie_word_embeddings": isinstance(model.embed_tokens, blocks.QuantizedEmbedding)
        and model.lm_head.weight.data_ptr() == model.embed_tokens.weight.data_ptr(),
        "quantization": {"group_size": 64, "bits": 4},
    }


def save_torch_lm(model, directory, shards=1):
    """Write `model` as an MLX-community-style 4-bit checkpoint directory."""
    os.makedirs(directory, exist_ok=True)
    config = model_config(model)
    tensors = {}
    if isinstance(model.embed_tokens, blocks.QuantizedEmbedding):
        tensors.update(_linear_tensors("model.embed_tokens", model.embed_tokens))
    else:
        tensors["model.embed_tokens.weight"] = model.embed_tokens.weight
    for index, layer in enumerate(model.layers):
        base = f"model.layers.{index}"
        for name in ("q_proj", "k_proj", "v_proj", "o_proj"):
            tensors.update(_linear_tensors(f"{base}.self_attn.{name}", getattr(layer.self_attn, name)))
        for name in ("gate_proj", "up_proj", "down_proj"):
            tensors.update(_linear_tensors(f"{base}.mlp.{name}", getattr(layer.mlp, name)))
        tensors[f"{base}.input_layernorm.weight"] = layer.input_layernorm.weight
        tensors[f"{base}.post_attention_layernorm.weight"] = layer.post_attention_layernorm.weight
    tensors["model.norm.weight"] = model.norm.weight
    if not config["tie_word_embeddings"]:
        tensors.update(_linear_tensors("lm_head", model.lm_head))
    with open(os.path.join(directory, "config.json"), "w") as handle:
        json.dump(config, handle, indent=2)
    names = sorted(tensors)
    if shards <= 1:
        write_safetensors(os.path.join(directory, "model.safetensors"), tensors, {"format": "mlx"})
        return config
    weight_map = {}
    for shard in range(shards):
        part = names[shard::shards]
        file_name = f"model-{shard + 1:05d}-of-{shards:05d}.safetensors"
        write_safetensors(os.path.join(directory, file_name), {n: tensors[n] for n in part}, {"format": "mlx"})
        weight_map.update({n: file_name for n in part})
    with open(os.path.join(directory, "model.safetensors.index.json"), "w") as handle:
        json.dump({"metadata": {}, "weight_map": weight_map}, handle, indent=2)
    return config


def _take_linear(tensors, prefix, device, group_size, bits):
    try:
        weight, scales, biases = (tensors[f"{prefix}.{part}"] for part in ("weight", "scales", "biases"))
    except KeyError as error:
        raise ValueError(f"checkpoint has no 4-bit triple for {prefix}: missing {error.args[0]}") from None
    if weight.dtype is not torch.uint32 or weight.ndim != 2:
        raise ValueError(f"{prefix}.weight must be uint32 [N, K/8], got {weight.dtype} {tuple(weight.shape)}")
    expected = (weight.shape[0], weight.shape[1] * 32 // bits // group_size)
    if tuple(scales.shape) != expected or tuple(biases.shape) != expected:
        raise ValueError(f"{prefix}: scales / biases must be {expected}, got {tuple(scales.shape)} / {tuple(biases.shape)}")
    bias = tensors.get(f"{prefix}.bias")
    move = lambda t: t.to(torch.bfloat16).to(device) if t.is_floating_point() else t.to(device)  # noqa: E731
    return blocks.QuantizedLinear(move(weight), move(scales), move(biases), group_size=group_size, bits=bits,
                                  bias=None if bias is None else move(bias))


def load_torch_lm(directory, device="cuda"):
    """Build a `blocks.TinyCausalLM` from an MLX-community-style 4-bit checkpoint directory.  The
    packed weights go to the device as they are in the file."""
    with open(os.path.join(directory, "config.json")) as handle:
        config = json.load(handle)
    quantization = config.get("quantization") or {}
    group_size, bits = quantization.get("group_size"), quantization.get("bits")
    if (group_size, bits) != (64, 4):
        raise ValueError(f"only 4-bit, group-size-64 checkpoints are supported, got bits={bits} group_size={group_size}")
    tensors = read_checkpoint_tensors(directory)
    heads, kv_heads = config["num_attention_heads"], config.get("num_key_value_heads") or config["num_attention_heads"]
    head_dim = config.get("head_dim") or config["hidden_size"] // heads
    eps, theta = config.get("rms_norm_eps", 1e-6), config.get("rope_theta", 10000.0)
    linear = lambda prefix: _take_linear(tensors, prefix, device, group_size, bits)  # noqa: E731
    norm = lambda name: blocks.RMSNorm(tensors[name].to(torch.bfloat16).to(device), eps)  # noqa: E731
    layers = []
    for index in range(config["num_hidden_layers"]):
        base = f"model.layers.{index}"
        attention = blocks.Attention(linear(f"{base}.self_attn.q_proj"), linear(f"{base}.self_attn.k_proj"),
                                     linear(f"{base}.self_attn.v_proj"), linear(f"{base}.self_attn.o_proj"), heads,
                                     kv_heads, head_dim, theta)
        mlp = blocks.GatedMLP(linear(f"{base}.mlp.gate_proj"), linear(f"{base}.mlp.up_proj"), linear(f"{base}.mlp.down_proj"))
        layers.append(blocks.DecoderBlock(norm(f"{base}.input_layernorm.weight"), attention,
                                          norm(f"{base}.post_attention_layernorm.weight"), mlp))
    if "model.embed_tokens.scales" in tensors:
        source = _take_linear(tensors, "model.embed_tokens", device, group_size, bits)
        embed = blocks.QuantizedEmbedding(source.weight, source.scales, source.biases, group_size=group_size, bits=bits)
    else:
        embed = torch.nn.Embedding.from_pretrained(tensors["model.embed_tokens.weight"].to(torch.bfloat16).to(device), freeze=True)
    if config.get("tie_word_embeddings") and "lm_head.weight" not in tensors:
        if not isinstance(embed, blocks.QuantizedEmbedding):
            raise ValueError("tied word embeddings need a quantised embedding to serve as the 4-bit lm_head")
        head = embed.as_linear()
    else:
        head = linear("lm_head")
    return blocks.TinyCausalLM(embed, layers, norm("model.norm.weight"), head, config["vocab_size"])
